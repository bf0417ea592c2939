"""Each kernel alone against a plain float64 reference written here, at sizes other than the
engine's: widths and vocabularies that are no power of two, odd head counts and groups, head
sizes in steps of 16.  Attention is fed shuffled block tables, a pool whose foreign pages and
unwritten cells hold NaN, and queries aimed at one far key so that a wrong cell would show."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------------------
# norms, embedding, activation
# ---------------------------------------------------------------------------------------------

def ref_rmsnorm(x, w, eps):
    x = x.double()
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()


@pytest.mark.parametrize("width", [120, 1000, 4096, 5000, 9000])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_plain_delta_parts_rows(width, out_dtype):
    from lgml_b200 import ops

    torch.manual_seed(width)
    n, eps = 7, 3e-6
    x0 = torch.randn(n, width) * 3
    w = 1 + 0.1 * torch.randn(width)
    tol = dict(atol=2e-6, rtol=2e-6) if out_dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    # plain
    x = x0.to(DEV)
    out = torch.empty(n, width, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, w.to(DEV), eps, out)
    assert torch.allclose(out.double().cpu(), ref_rmsnorm(x0, w, eps), **tol)
    # residual add of a bfloat16 delta, written back
    delta = torch.randn(n, width).to(torch.bfloat16)
    x = x0.to(DEV)
    ops.rmsnorm(x, w.to(DEV), eps, out, delta=delta.to(DEV))
    want_x = x0.double() + delta.double()
    assert torch.allclose(x.double().cpu(), want_x, atol=1e-6, rtol=1e-6)
    assert torch.allclose(out.double().cpu(), ref_rmsnorm(want_x, w, eps), **tol)
    # partial sums of a product cut along K, with a bias, and a row gather (x untouched)
    parts = torch.randn(6, n, width)
    bias = torch.randn(width)
    rows = torch.tensor([5, 0, 5, 2], dtype=torch.int32)
    x = x0.to(DEV)
    outr = torch.empty(4, width, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, w.to(DEV), eps, outr, delta=ops.Partials(parts.to(DEV), bias.to(DEV)), rows=rows.to(DEV))
    want_x = x0.double() + parts.double().sum(0) + bias.double()
    assert torch.equal(x.cpu(), x0)
    assert torch.allclose(outr.double().cpu(), ref_rmsnorm(want_x[rows.long()], w, eps), **tol)
    # the same sum without the row list is written back
    ops.rmsnorm(x, w.to(DEV), eps, out, delta=ops.Partials(parts.to(DEV), bias.to(DEV)))
    assert torch.allclose(x.double().cpu(), want_x, atol=1e-5, rtol=1e-6)


@pytest.mark.parametrize("width", [777, 1500, 4096, 5000, 9000, 20000])
def test_rmsnorm_row_does_not_depend_on_the_batch(width):
    """A row among many (a block per row) and the same row alone (spread over a cluster when it
    is wide) come out with the same bits, with and without partial sums added first."""
    from lgml_b200 import ops

    torch.manual_seed(0)
    w = torch.rand(width, device=DEV) + 0.5
    x = torch.randn(100, width, device=DEV)
    a = torch.empty(100, width, device=DEV)
    b = torch.empty(1, width, device=DEV)
    ops.rmsnorm(x.clone(), w, 1e-5, a)
    ops.rmsnorm(x[41:42].clone(), w, 1e-5, b)
    assert torch.equal(a[41], b[0])
    parts = torch.randn(5, 100, width, device=DEV)
    bias = torch.randn(width, device=DEV)
    xa, xb = x.clone(), x[41:42].clone()
    ops.rmsnorm(xa, w, 1e-5, a, delta=ops.Partials(parts, bias))
    ops.rmsnorm(xb, w, 1e-5, b, delta=ops.Partials(parts[:, 41:42].contiguous(), bias))
    assert torch.equal(a[41], b[0]) and torch.equal(xa[41], xb[0])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_rows(dtype):
    from lgml_b200 import ops

    torch.manual_seed(1)
    table = torch.randn(331, 120).to(dtype)
    ids = torch.tensor([0, 330, 17, 17, 200], dtype=torch.int32)
    out = torch.empty(5, 120, device=DEV)
    st = status()
    ops.embed_rows(table.to(DEV), ids.to(DEV), out, st)
    assert torch.equal(out.cpu(), table[ids.long()].float()) and int(st.item()) == 0
    # an id outside the table is flagged and read as zeros, never out of bounds
    ops.embed_rows(table.to(DEV), torch.tensor([3, 331, -1, 4, 5], dtype=torch.int32, device=DEV), out, st)
    assert int(st.item()) == 1 and float(out[1].abs().sum()) == 0.0 and float(out[2].abs().sum()) == 0.0


@pytest.mark.parametrize("paired", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(paired, dtype):
    from lgml_b200 import ops

    torch.manual_seed(2)
    g, u = torch.randn(5, 200).to(dtype), torch.randn(5, 200).to(dtype)
    gu = torch.stack([g, u], 2).reshape(5, 400) if paired else torch.cat([g, u], 1)
    out = torch.empty(5, 200, dtype=dtype, device=DEV)
    ops.silu_mul(gu.contiguous().to(DEV), out, paired=paired)
    want = g.double() * torch.sigmoid(g.double()) * u.double()
    tol = dict(atol=1e-6, rtol=1e-6) if dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    assert torch.allclose(out.double().cpu(), want, **tol)


def test_l2_ahead_touches_nothing_and_refuses_a_ragged_address():
    from lgml_b200 import ops

    w = torch.randn(3000, 1111, device=DEV).to(torch.bfloat16)      # a size that is no multiple of a chunk
    before = w.clone()
    for n in (None, 0, 15, 16, 40_000, w.numel() * 2 + 999):
        ops.l2_ahead(w, n)
        ops.l2_ahead(w, n, keep=False)
    torch.cuda.synchronize()
    assert torch.equal(w, before)
    with pytest.raises(ops.KernelError, match="16-byte"):
        ops.l2_ahead(w.view(-1)[1:], 64)


def test_fill_normal_is_seeded():
    from lgml_b200 import ops

    a = torch.empty(1 << 20, device=DEV)
    b = torch.empty(1 << 20, device=DEV)
    ops.fill_normal(a, 1.0, 0.02, 7)
    ops.fill_normal(b, 1.0, 0.02, 7)
    assert torch.equal(a, b)
    ops.fill_normal(b, 1.0, 0.02, 8)
    assert not torch.equal(a, b)
    assert abs(float(a.mean()) - 1.0) < 1e-4 and abs(float(a.std()) - 0.02) < 2e-4
    z = (a - 1.0) / 0.02
    assert abs(float((z.abs() < 1).float().mean()) - 0.6827) < 5e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fill_normal_draws_the_host_generator_bit_for_bit(dtype):
    """One generator on both sides: the device's fill equals ``fill_normal_host`` in every bit,
    over several keys, sizes that end inside a block of threads, and both kinds of init."""
    from lgml_b200 import ops
    from lgml_b200.weights.random_init import fill_normal_host, tensor_key

    for key, n, mean, sd in ((tensor_key(0, "model.embed_tokens.weight"), 1 << 18, 0.0, 0.02), (tensor_key(3, "x"), 100003, 1.0, 0.02),
                             (0xFFFFFFFFFFFFFFFF, 4097, -0.5, 1.0), (1, 1, 0.0, 1.0)):
        dev = torch.empty(n, dtype=dtype, device=DEV)
        ops.fill_normal(dev, mean, sd, key)
        host = fill_normal_host((n,), mean, sd, key).to(dtype)
        assert torch.equal(dev.cpu().view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                           host.view(torch.int16 if dtype == torch.bfloat16 else torch.int32)), (key, n)


# ---------------------------------------------------------------------------------------------
# matrix products
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 200, 120), (70, 331, 257), (3, 1000, 96)])
def test_gemm_f32_is_exact_and_batch_invariant(M, N, K):
    from lgml_b200 import ops

    torch.manual_seed(M * N)
    a, w, b = torch.randn(M, K), torch.randn(N, K), torch.randn(N)
    out = torch.empty(M, N, device=DEV)
    ops.gemm_f32(a.to(DEV), w.to(DEV), out, b.to(DEV))
    want = a.double() @ w.double().t() + b.double()
    assert torch.allclose(out.double().cpu(), want, atol=1e-5 * math.sqrt(K), rtol=1e-6)
    one = torch.empty(1, N, device=DEV)
    ops.gemm_f32(a[M - 1:].contiguous().to(DEV), w.to(DEV), one, b.to(DEV))
    assert torch.equal(one[0], out[M - 1])          # a row's bits do not depend on the other rows


@pytest.mark.parametrize("M,N,K,bias,f32,splits", [
    (1, 128, 64, False, False, None), (8, 331 * 8, 120, True, True, None), (5, 200, 192, True, False, 3),
    (64, 1000, 1096, True, True, 4), (100, 320, 96, False, False, None), (129, 520, 264, True, False, None),
    (300, 648, 200, True, True, None), (700, 1200, 520, False, False, None),
    # 512 rows and more: pairs of CTAs on 256 x 256 tiles (edges in every direction, several tiles per pair)
    (512, 256, 64, False, False, None), (777, 1000, 328, True, True, None), (1500, 40 * 256 + 8, 136, True, False, None),
    # narrower tiles where 256 columns would leave pairs idle: 192 (512 x 6144: 64 tiles) and 128 (512 x 4096)
    (512, 6144 - 16, 200, True, False, None), (500, 4000, 136, False, True, None),
    # 65 to 511 rows on pairs too; few tiles: K in ranges of whole 128-element stages, summed by the reduce kernel
    (65, 256, 2048 + 8, True, False, None), (128, 520, 3000, False, True, None), (200, 384, 1096, True, True, 3), (300, 256, 640, False, False, 5),
])
def test_gemm_tcgen05(M, N, K, bias, f32, splits):
    from lgml_b200 import ops

    torch.manual_seed(M + N + K)
    x = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.1).to(torch.bfloat16)
    b = torch.randn(N) if bias else None
    st = status()
    out = torch.full((M, N), float("nan"), dtype=torch.float32 if f32 else torch.bfloat16, device=DEV)
    ops.gemm_tcgen05(x.to(DEV), w.to(DEV), out, None if b is None else b.to(DEV), st, n_splits=splits)
    want = x.double() @ w.double().t() + (b.double() if bias else 0)
    scale = float(want.abs().max())
    err = float((out.double().cpu() - want).abs().max())
    assert int(st.item()) == 0
    assert err <= scale * (5e-5 if f32 else 6e-3), (err, scale)


def test_gemm_tcgen05_on_single_ctas_when_pairs_are_switched_off():
    """``LGML_GEMM_PAIR=0`` (read once per process, so a process of its own): products of more
    than 64 tokens on single CTAs, the weights as the tile's rows up to 256 tokens and persistent
    128 x 256 tiles beyond."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    code = """
import torch
from lgml_b200 import ops
st = torch.zeros(1, dtype=torch.int32, device="cuda:0")
for M, N, K, gated in [(100, 320, 96, False), (129, 520, 264, False), (256, 300, 200, True), (300, 648, 200, False), (700, 1200, 520, True)]:
    torch.manual_seed(M)
    x = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.1).to(torch.bfloat16)
    if gated:
        got = ops.gemm_bf16_swiglu(x.cuda(), w.cuda(), None, st).double().cpu()
        y = x.double() @ w.double().t()
        want = y[:, 0::2] * torch.sigmoid(y[:, 0::2]) * y[:, 1::2]
    else:
        out = torch.empty(M, N, dtype=torch.float32, device="cuda:0")
        got = ops.gemm_tcgen05(x.cuda(), w.cuda(), out, None, st).double().cpu()
        want = x.double() @ w.double().t()
    assert float((got - want).abs().max()) <= 6e-3 * float(want.abs().max()), (M, N, K)
assert int(st.item()) == 0
assert ops.tcgen05_splits(300, 256, 640) == 1          # the pairs' K ranges are off too
print("ok")
"""
    root = Path(__file__).resolve().parent.parent
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=root, env={**os.environ, "LGML_GEMM_PAIR": "0"}, timeout=300)
    assert p.returncode == 0 and p.stdout.strip().endswith("ok"), p.stdout + p.stderr


def test_gemm_tcgen05_gated_epilogue_and_partials():
    from lgml_b200 import ops

    torch.manual_seed(5)
    st = status()
    for M, F, K in [(6, 100, 96), (100, 331, 264), (128, 260, 1096), (300, 176, 120), (640, 300, 200)]:
        x = torch.randn(M, K).to(torch.bfloat16)
        wg, wu = (torch.randn(F, K) * 0.1).to(torch.bfloat16), (torch.randn(F, K) * 0.1).to(torch.bfloat16)
        bg, bu = torch.randn(F), torch.randn(F)
        pairs = torch.stack([wg, wu], 1).reshape(2 * F, K).contiguous()
        bp = torch.stack([bg, bu], 1).reshape(2 * F).contiguous()
        out = ops.gemm_bf16_swiglu(x.to(DEV), pairs.to(DEV), bp.to(DEV), st)
        g = x.double() @ wg.double().t() + bg.double()
        u = x.double() @ wu.double().t() + bu.double()
        want = g * torch.sigmoid(g) * u
        assert float((out.double().cpu() - want).abs().max()) <= 6e-3 * float(want.abs().max())
    x = torch.randn(9, 520).to(torch.bfloat16)
    w = (torch.randn(200, 520) * 0.1).to(torch.bfloat16)
    b = torch.randn(200)
    pr = ops.gemm_tcgen05(x.to(DEV), w.to(DEV), None, b.to(DEV), st, n_splits=3, partials_ok=True)
    assert isinstance(pr, ops.Partials) and pr.data.shape == (3, 9, 200)
    want = x.double() @ w.double().t() + b.double()
    assert float((pr.sum().double().cpu() - want).abs().max()) <= 5e-5 * float(want.abs().max())
    # the same from pairs of CTAs (more than 64 tokens): the K ranges the kernel library chooses
    x = torch.randn(130, 4096 + 64).to(torch.bfloat16)
    w = (torch.randn(300, 4096 + 64) * 0.1).to(torch.bfloat16)
    b = torch.randn(300)
    pr = ops.gemm_tcgen05(x.to(DEV), w.to(DEV), None, b.to(DEV), st, partials_ok=True)
    assert isinstance(pr, ops.Partials) and pr.data.shape[0] == ops.tcgen05_splits(130, 300, 4096 + 64) > 1
    want = x.double() @ w.double().t() + b.double()
    assert float((pr.sum().double().cpu() - want).abs().max()) <= 5e-5 * float(want.abs().max())
    assert int(st.item()) == 0


def test_gemm_bf16_falls_back_when_tma_cannot_take_the_operands():
    from lgml_b200 import ops

    x = torch.randn(4, 100).to(torch.bfloat16).to(DEV)        # a row of 200 bytes: no multiple of 16
    w = torch.randn(50, 100).to(torch.bfloat16).to(DEV)
    assert not ops.tcgen05_supports(x, w)
    y = ops.gemm_bf16(x, w, torch.float32, status=status())
    assert torch.allclose(y.double().cpu(), x.double().cpu() @ w.double().cpu().t(), atol=1e-2, rtol=1e-2)


# ---------------------------------------------------------------------------------------------
# rotary encoding and cache write
# ---------------------------------------------------------------------------------------------

def ref_rope(x, pos, inv_freq, pairing, n_rot):
    x = x.double().clone()
    ang = pos.double()[:, None] * inv_freq.double()[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    if pairing == "adjacent":
        a, b = x[..., 0:n_rot:2].clone(), x[..., 1:n_rot:2].clone()
        x[..., 0:n_rot:2], x[..., 1:n_rot:2] = a * c - b * s, a * s + b * c
    else:
        h = n_rot // 2
        a, b = x[..., :h].clone(), x[..., h:n_rot].clone()
        x[..., :h], x[..., h:n_rot] = a * c - b * s, a * s + b * c
    return x


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pairing,n_rot,from_parts", [("half", 48, False), ("adjacent", 48, False), ("half", 32, False), ("half", 48, True), ("half", 0, False)])
@pytest.mark.parametrize("lens", [[3, 70, 1], [3, 5, 1]])     # many tokens take the kernel with 16-byte accesses, few the other
def test_rope_kv_write(dtype, pairing, n_rot, from_parts, lens):
    from lgml_b200 import ops

    torch.manual_seed(3)
    H, G, D, page = 5, 5 if n_rot == 32 else 1, 48, 64
    pos0 = [62, 0, 127]                                # the first request crosses a page edge
    n = sum(lens)
    positions = torch.tensor([p + i for p, ln in zip(pos0, lens) for i in range(ln)], dtype=torch.int32)
    seq_of = torch.tensor([s for s, ln in enumerate(lens) for _ in range(ln)], dtype=torch.int32)
    table = torch.tensor([[7, 2, -1], [4, 9, -1], [0, 5, -1]], dtype=torch.int32)
    inv_freq = torch.tensor([10000.0 ** (-2.0 * i / max(n_rot, 2)) for i in range(max(n_rot // 2, 1))], dtype=torch.float32)
    width = (H + 2 * G) * D
    st = status()
    k_pages = torch.full((12, G, page, D), float("nan"), dtype=dtype, device=DEV)
    v_pages = torch.full((12, G, page, D), float("nan"), dtype=dtype, device=DEV)
    if from_parts:
        parts = torch.randn(3, n, width)
        bias = torch.randn(width)
        full = (parts.double().sum(0) + bias.double())
        q = ops.rope_kv_write(ops.Partials(parts.to(DEV), bias.to(DEV)), positions.to(DEV), seq_of.to(DEV), table.to(DEV), inv_freq.to(DEV),
                              n_rot, pairing, k_pages, v_pages, H, G, D, st)
    else:
        qkv = torch.randn(n, width).to(dtype)
        full = qkv.double()
        dev_qkv = qkv.to(DEV)
        q = ops.rope_kv_write(dev_qkv, positions.to(DEV), seq_of.to(DEV), table.to(DEV), inv_freq.to(DEV), n_rot, pairing,
                              k_pages, v_pages, H, G, D, st)
    assert int(st.item()) == 0
    tol = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=1e-2)
    want_q = ref_rope(full[:, : H * D].reshape(n, H, D), positions, inv_freq[: n_rot // 2], pairing, n_rot)
    want_k = ref_rope(full[:, H * D:(H + G) * D].reshape(n, G, D), positions, inv_freq[: n_rot // 2], pairing, n_rot)
    want_v = full[:, (H + G) * D:].reshape(n, G, D)
    assert torch.allclose(q.double().cpu().reshape(n, H, D), want_q, **tol)
    kc, vc = k_pages.double().cpu(), v_pages.double().cpu()
    written = torch.zeros(12, page, dtype=torch.bool)
    for t in range(n):
        p = int(positions[t])
        pg = int(table[int(seq_of[t]), p // page])
        assert torch.allclose(kc[pg, :, p % page, :], want_k[t], **tol)
        assert torch.allclose(vc[pg, :, p % page, :], want_v[t], **tol)
        written[pg, p % page] = True
    assert bool(torch.isnan(kc.permute(0, 2, 1, 3)[~written]).all())           # no other cell was touched
    assert bool(torch.isnan(vc.permute(0, 2, 1, 3)[~written]).all())


@pytest.mark.parametrize("lens", [[3, 2], [40, 2]])      # both kernels
def test_rope_angles_at_far_positions(lens):
    """Positions near 100,000 and near 2^24 - 1: with the float64 table's remainders beside the
    float32 frequencies the rotation is right to a few float32 roundings; a single float32
    product pos * frequency would be off by thousandths of a radian there (by a radian at 2^24)."""
    from lgml_b200 import ops

    torch.manual_seed(5)
    H, G, D, page, n_rot = 3, 1, 32, 64, 32
    pos0 = [99_990, (1 << 24) - 70]
    n = sum(lens)
    positions = torch.tensor([p + i for p, ln in zip(pos0, lens) for i in range(ln)], dtype=torch.int32)
    seq_of = torch.tensor([s for s, ln in enumerate(lens) for _ in range(ln)], dtype=torch.int32)
    width_tab = (1 << 24) // page
    table = torch.zeros(2, width_tab, dtype=torch.int32)                # every block of both requests is page 0 or 1
    table[1] = 1
    exact = torch.tensor([500000.0 ** (-2.0 * i / n_rot) / (1.0 + 0.37 * i) for i in range(n_rot // 2)], dtype=torch.float64)
    hi = exact.float()
    both = torch.stack([hi, (exact - hi.double()).float()])
    qkv = torch.randn(n, (H + 2 * G) * D).to(torch.bfloat16 if lens[0] > 32 else torch.float32)
    want_q = ref_rope(qkv.double()[:, : H * D].reshape(n, H, D), positions, exact, "half", n_rot)
    err = {}
    for name, freq in (("with remainders", both), ("float32 alone", hi)):
        st = status()
        k_pages = torch.zeros((2, G, page, D), dtype=qkv.dtype, device=DEV)
        q_out = torch.empty(n, H * D, dtype=qkv.dtype, device=DEV)
        ops.rope_kv_write(qkv.to(DEV), positions.to(DEV), seq_of.to(DEV), table.to(DEV), freq.to(DEV), n_rot, "half", k_pages,
                          torch.zeros_like(k_pages), H, G, D, st, q_out=q_out)
        assert int(st.item()) == 0
        err[name] = float((q_out.double().cpu().reshape(n, H, D) - want_q).abs().max())
    if qkv.dtype == torch.float32:
        assert err["with remainders"] < 5e-6 and err["float32 alone"] > 1e-3, err
    else:
        assert err["with remainders"] < 3e-2 and err["float32 alone"] > 1e-1, err     # bfloat16 rounds q itself to 2^-9


# ---------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------

def make_attention_case(seed, H, G, D, kv_lens, q_lens, dtype, n_pages=40, aim=True):
    """Requests with kv_lens cached tokens of which the last q_lens are this step's queries.
    Pages are shuffled; every cell no request owns holds NaN."""
    g = torch.Generator().manual_seed(seed)
    page = 64
    perm = torch.randperm(n_pages, generator=g).tolist()
    k_pages = torch.full((n_pages, G, page, D), float("nan"))
    v_pages = torch.full((n_pages, G, page, D), float("nan"))
    width = max(-(-max(kv_lens) // page), 1) + 1
    table = torch.full((len(kv_lens), width), -1, dtype=torch.int32)
    ks, vs, qs, positions, seq_of = [], [], [], [], []
    for s, (n, nq) in enumerate(zip(kv_lens, q_lens)):
        k, v = torch.randn(n, G, D, generator=g), torch.randn(n, G, D, generator=g)
        q = torch.randn(nq, H, D, generator=g)
        if aim and n > 3:
            # aim the last query of every head at one far key: its score stands out by ~12
            far = 1 if n < 70 else n - 67
            for h in range(H):
                kk = k[far, h // (H // G)]
                q[-1, h] = kk / kk.norm() * 12.0 * math.sqrt(D) / kk.norm()
        k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
        for b in range(-(-n // page)):
            table[s, b] = perm.pop()
            rows = slice(b * page, min((b + 1) * page, n))
            k_pages[table[s, b], :, : rows.stop - rows.start] = k[rows].transpose(0, 1).float()
            v_pages[table[s, b], :, : rows.stop - rows.start] = v[rows].transpose(0, 1).float()
        ks.append(k.double()); vs.append(v.double()); qs.append(q.double())
        positions += list(range(n - nq, n))
        seq_of += [s] * nq
    q_all = torch.cat([q.reshape(q.shape[0], H * D) for q in qs]).to(dtype)
    return dict(q=q_all, k_pages=k_pages.to(dtype), v_pages=v_pages.to(dtype), table=table, positions=torch.tensor(positions, dtype=torch.int32),
                seq_of=torch.tensor(seq_of, dtype=torch.int32), ks=ks, vs=vs, qs=qs, H=H, G=G, D=D, kv_lens=kv_lens, q_lens=q_lens)


def ref_attention(case, scale, window):
    outs = []
    H, G, D = case["H"], case["G"], case["D"]
    for k, v, q, n, nq in zip(case["ks"], case["vs"], case["qs"], case["kv_lens"], case["q_lens"]):
        o = torch.empty(nq, H, D, dtype=torch.float64)
        for i in range(nq):
            p = n - nq + i
            lo = max(0, p - window + 1) if window else 0
            for h in range(H):
                s = (k[lo:p + 1, h // (H // G)] @ q[i, h]) * scale
                o[i, h] = torch.softmax(s, 0) @ v[lo:p + 1, h // (H // G)]
        outs.append(o.reshape(nq, H * D))
    return torch.cat(outs)


class FakeBatch:
    def __init__(self, case):
        self.positions, self.seq_of_token = case["positions"].to(DEV), case["seq_of"].to(DEV)
        self.max_q_len, self.max_kv_len = max(case["q_lens"]), max(case["kv_lens"])
        self.seq_lens = case["q_lens"]
        self.decode_splits = None

    def attention_tiles(self, tt):
        rows, start = [], 0
        for s, n in enumerate(self.seq_lens):
            rows += [(s, start + t0, min(tt, n - t0), 0) for t0 in range(0, n, tt)]
            start += n
        return torch.tensor(rows, dtype=torch.int32, device=DEV)


ATT_SHAPES = [(4, 4, 16), (6, 2, 32), (5, 5, 48), (8, 1, 64), (12, 4, 128), (9, 1, 80)]


def run_attention(kind, case, window, n_splits=None):
    from lgml_b200 import ops

    st = status()
    H, D = case["H"], case["D"]
    scale = D ** -0.5
    q = case["q"].to(DEV)
    out = torch.full_like(q, float("nan"))
    kp, vp, tab = case["k_pages"].to(DEV), case["v_pages"].to(DEV), case["table"].to(DEV)
    b = FakeBatch(case)
    if kind == "ref":
        ops.paged_attention_ref(q, b.positions, b.seq_of_token, tab, kp, vp, out, H, scale, window, st)
    elif kind == "decode":
        ops.decode_attention(q, b.positions, b.seq_of_token, tab, kp, vp, out, H, scale, window, st, n_splits)
    elif kind == "prefill_tc":
        tiles = b.attention_tiles(ops.prefill_tc_tile_tokens(H, case["G"]))
        ops.prefill_attention_tc(q, b.positions, tiles, tab, kp, vp, out, H, scale, window, st)
    elif kind == "prefill_twin":
        tiles = b.attention_tiles(ops.prefill_twin_tile_tokens(H, case["G"]))
        ops.prefill_attention_twin(q, b.positions, tiles, tab, kp, vp, out, H, scale, window, st)
    else:
        tiles = b.attention_tiles(ops.prefill_tile_tokens(H, case["G"]))
        ops.prefill_attention(q, b.positions, tiles, tab, kp, vp, out, H, scale, window, st)
    assert int(st.item()) == 0
    return out.double().cpu(), ref_attention(case, scale, window)


@pytest.mark.parametrize("H,G,D", ATT_SHAPES + [(2, 2, 256), (3, 1, 40)])
@pytest.mark.parametrize("dtype,window", [(torch.float32, 0), (torch.float32, 37), (torch.bfloat16, 0)])
def test_attention_ref_kernel(H, G, D, dtype, window):
    case = make_attention_case(1, H, G, D, kv_lens=[200, 1, 65, 130], q_lens=[200, 1, 2, 7], dtype=dtype)
    got, want = run_attention("ref", case, window)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    assert torch.isfinite(got).all() and torch.allclose(got, want, **tol)


@pytest.mark.parametrize("H,G,D", ATT_SHAPES + [(16, 1, 32), (4, 2, 256)])
@pytest.mark.parametrize("window,n_splits", [(0, 1), (0, 5), (100, 3), (0, 8), (0, 11), (100, 9)])
def test_attention_decode_kernel(H, G, D, window, n_splits):
    case = make_attention_case(2, H, G, D, kv_lens=[700, 64, 1, 333, 129, 65], q_lens=[1, 1, 1, 3, 1, 2], dtype=torch.bfloat16)
    got, want = run_attention("decode", case, window, n_splits)
    assert torch.isfinite(got).all() and torch.allclose(got, want, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("H,G,D", ATT_SHAPES + [(3, 3, 112), (16, 1, 64)])
@pytest.mark.parametrize("window", [0, 90])
@pytest.mark.parametrize("kind", ["prefill", "prefill_tc"])
def test_attention_prefill_kernel(H, G, D, window, kind):
    case = make_attention_case(3, H, G, D, kv_lens=[300, 70, 1, 129, 64], q_lens=[300, 33, 1, 65, 2], dtype=torch.bfloat16)
    got, want = run_attention(kind, case, window)
    assert torch.isfinite(got).all() and torch.allclose(got, want, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("H,G,D", [(8, 1, 64), (12, 4, 128), (16, 1, 64), (6, 2, 128), (3, 3, 64), (5, 5, 128), (32, 2, 64)])
@pytest.mark.parametrize("window", [0, 90, 200])
def test_attention_prefill_twin_kernel(H, G, D, window):
    """Two tiles per CTA, two pages per step: full and partly filled tiles, a second tile with
    one token, steps with one page, portions that start inside a page and far from it."""
    case = make_attention_case(3, H, G, D, kv_lens=[300, 70, 1, 129, 64, 515, 260], q_lens=[300, 33, 1, 65, 2, 130, 257], dtype=torch.bfloat16)
    got, want = run_attention("prefill_twin", case, window)
    assert torch.isfinite(got).all() and torch.allclose(got, want, atol=3e-2, rtol=2e-2)


def test_attention_prefill_twin_many_launches_never_wait_out():
    """A wait on an mbarrier that runs out sets the status word and costs about a second; a thread
    that comes late to a barrier of two phases did that once in some hundred launches.  Full
    tiles, a last page that is partly filled, and launches back to back."""
    from lgml_b200 import ops
    import time

    H, G, D, T = 8, 2, 128, 1000
    st = status()
    n_pages = -(-T // 64)
    k = torch.randn(n_pages, G, 64, D, device=DEV).to(torch.bfloat16)
    v = torch.randn(n_pages, G, 64, D, device=DEV).to(torch.bfloat16)
    q = torch.randn(T, H * D, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    table = torch.randperm(n_pages).to(torch.int32).reshape(1, n_pages).to(DEV)
    tt = ops.prefill_twin_tile_tokens(H, G)
    tiles = torch.tensor([(0, t0, min(tt, T - t0), 0) for t0 in reversed(range(0, T, tt))], dtype=torch.int32, device=DEV)
    ops.prefill_attention_twin(q, positions, tiles, table, k, v, out, H, D ** -0.5, 0, st)
    first = out.clone()
    torch.cuda.synchronize()
    t0 = time.time()
    for _ in range(1500):
        ops.prefill_attention_twin(q, positions, tiles, table, k, v, out, H, D ** -0.5, 0, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and time.time() - t0 < 0.9 and torch.equal(out, first)


def test_attention_finds_the_far_key():
    """The aimed query's output is that key's value, in every kernel."""
    case = make_attention_case(4, 4, 2, 64, kv_lens=[500], q_lens=[1], dtype=torch.bfloat16)
    far = 500 - 67
    for kind, splits in (("ref", None), ("decode", 4), ("prefill", None), ("prefill_tc", None), ("prefill_twin", None)):
        got, _ = run_attention(kind, case, 0, splits)
        for h in range(4):
            v_far = case["vs"][0][far, h // 2]
            assert float((got[0, h * 64:(h + 1) * 64] - v_far).abs().max()) < 0.15, kind


# ---------------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------------

def test_argmax_lowest_index_wins_and_odd_vocabulary():
    from lgml_b200 import ops

    torch.manual_seed(6)
    logits = torch.randn(5, 128257)
    logits[0, 77] = logits[0, 100000] = 50.0          # a tie
    logits[1, 128256] = 60.0                          # the last column
    logits[2] = float("-inf")
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax_rows(logits.to(DEV), out)
    got = out.cpu().tolist()
    assert got[0] == 77 and got[1] == 128256 and got[2] == 0
    assert got[3:] == torch.argmax(logits[3:], 1).tolist()


def test_sample_rows_matches_the_host_sampler():
    from lgml_b200 import ops
    from lgml_b200.sampling import Sampler, SamplingParams

    torch.manual_seed(7)
    V, R = 5003, 64
    logits = torch.randn(R, V) * 3
    temps = [0.0, 0.7, 1.0, 1.5] * (R // 4)
    samplers = [Sampler(SamplingParams.neutral(t, seed=100 + i)) for i, t in enumerate(temps)]
    twins = [Sampler(SamplingParams.neutral(t, seed=100 + i)) for i, t in enumerate(temps)]
    us = [0.0 if t <= 0 else s.uniform() for s, t in zip(samplers, temps)]
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.sample_rows(logits.to(DEV), torch.tensor(temps, device=DEV), torch.tensor(us, dtype=torch.float64, device=DEV), out)
    host = [tw.sample(logits[i].numpy()) for i, tw in enumerate(twins)]
    assert out.cpu().tolist() == host


@pytest.mark.parametrize("V,k", [(300, 1), (300, 40), (5000, 128), (128256, 40), (1024, 7)])
def test_topk_rows(V, k):
    """The k best of each row in the sampler's order (logit descending, id ascending), with
    ties, rows of one value, infinities and NaN."""
    import numpy as np
    from lgml_b200 import ops

    g = torch.Generator().manual_seed(V + k)
    rows = [torch.randn(V, generator=g) * 3,
            torch.randint(-3, 4, (V,), generator=g).float(),            # many ties
            torch.full((V,), 1.25),                                      # one value: the lowest ids win
            torch.randn(V, generator=g)]
    rows[3][::7] = float("-inf")
    rows[3][5] = float("nan")
    rows[3][11] = float("inf")
    x = torch.stack(rows)
    vals, ids = ops.topk_rows(x.to(DEV), k)
    vals, ids = vals.cpu().numpy(), ids.cpu().numpy()
    for r in range(x.shape[0]):
        l = x[r].numpy().astype(np.float64)
        l[np.isnan(l)] = -np.inf                                         # NaN sorts last (with -inf, by id)
        order = np.lexsort((np.arange(V), -l))[:k]
        nan_free = ~np.isnan(x[r].numpy()[order])
        assert np.array_equal(ids[r][nan_free], order[nan_free]), (r, ids[r][:8], order[:8])
        assert np.array_equal(vals[r][nan_free], x[r].numpy()[order][nan_free])


def test_sampler_edits_match_the_host_sampler():
    """Bias and history penalties on the device give, bit for bit, the logits the host sampler
    works on."""
    import numpy as np
    from lgml_b200 import ops
    from lgml_b200.sampling import Sampler, SamplingParams

    g = torch.Generator().manual_seed(8)
    V = 777
    x = (torch.randn(3, V, generator=g) * 4)
    samplers = [Sampler(SamplingParams(seed=1, repeat_penalty=1.3, frequency_penalty=0.25, presence_penalty=0.5, repeat_last_n=8, logit_bias={4: 1.5, 700: -3.0})),
                Sampler(SamplingParams(seed=2)),
                Sampler(SamplingParams(seed=3, repeat_penalty=0.8, logit_bias={0: 0.125}))]
    for s, hist in zip(samplers, ([5, 4, 5, 5, 9, 700, 3, 3, 3, 12], [1, 2, 3], [0, 0, 776])):
        for t in hist:
            s.accept(t)
    import struct
    per_row = [s.device_edits() for s in samplers]
    stride = 2 + 2 * max(len(b) + len(h) for b, h, _ in per_row)
    edits = torch.zeros((3, stride), dtype=torch.int32)
    params = torch.empty((3, 3), dtype=torch.float32)
    for i, (bias, hist, pen) in enumerate(per_row):
        flat = [len(bias), len(hist)]
        for t, b in bias:
            flat += [t, struct.unpack("<i", struct.pack("<f", b))[0]]
        for t, c in hist:
            flat += [t, c]
        edits[i, :len(flat)] = torch.tensor(flat, dtype=torch.int32)
        params[i] = torch.tensor(pen, dtype=torch.float32)
    got = ops.sampler_edits(x.clone().to(DEV), edits.to(DEV), params.to(DEV)).cpu().numpy()
    for i, s in enumerate(samplers):
        s.p.temperature = 0.0                      # sample() then stops after bias and penalties
        s.sample(x[i].numpy())
        assert np.array_equal(got[i], s.last_logits), i


@pytest.mark.parametrize("k", [1, 40, 128])
def test_sample_candidates_matches_the_host_sampler(k):
    """top_p, min_p, temperature and the draw on top_k's candidates, on the device: the ids of
    the host sampler given the same uniform numbers, over flat and peaked rows and every
    combination of the three options being on or off; temperature 0 takes the first candidate."""
    import math

    import numpy as np
    from lgml_b200 import ops
    from lgml_b200.sampling import Sampler, SamplingParams

    V, n = 5000, 96
    g = torch.Generator().manual_seed(k)
    scale = torch.tensor([0.3, 1.0, 4.0, 12.0]).repeat(n // 4)[:, None]
    x = torch.randn(n, V, generator=g) * scale
    x[5, :] = 0.5                                                       # one value everywhere
    opts = [dict(top_p=tp, min_p=mp, temperature=T) for tp in (1.0, 0.95, 0.3) for mp in (0.0, 0.05, 0.6) for T in (1.0, 0.8, 2.5)]
    chains = [SamplingParams(seed=100 + r, top_k=k, **opts[r % len(opts)]) for r in range(n)]
    chains[7] = SamplingParams(seed=7, temperature=0.0)
    vals, ids = ops.topk_rows(x.to(DEV), k)
    params = torch.tensor([[c.top_p, math.log(c.min_p) if c.min_p > 0 else -math.inf, c.temperature] for c in chains], dtype=torch.float32)
    us = torch.tensor([0.0 if c.greedy else Sampler(c).uniform() for c in chains], dtype=torch.float64)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample_candidates(vals, ids, params.to(DEV), us.to(DEV), out)
    got = out.cpu().tolist()
    vals, ids = vals.cpu().numpy(), ids.cpu().numpy()
    want = [int(ids[r][0]) if c.greedy else Sampler(c).sample_candidates(ids[r], vals[r]) for r, c in enumerate(chains)]
    assert got == want, [(r, a, b) for r, (a, b) in enumerate(zip(got, want)) if a != b]
    assert len(set(got)) > 1 if k > 1 else True
