"""ctypes bindings of the host library (``csrc/host/lgml_host.c``): the safetensors reader and
the sampler, in C as in mischief/lgml (``src/safetensors.c``, ``src/sample.c``).  Built with the
system's C compiler the first time something needs it; there is no other implementation."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_uint64, c_void_p
from typing import Optional

from . import csrc

ST_MAX_NAME, ST_MAX_RANK = 63, 4
ST_DTYPES = ("F64", "F32", "F16", "BF16", "I64", "I32", "I16", "I8")


class StEntry(Structure):
    _fields_ = [("name", c_char * (ST_MAX_NAME + 1)), ("dtype", c_int32), ("rank", c_int32), ("shape", c_int64 * ST_MAX_RANK),
                ("begin", c_int64), ("end", c_int64)]


class SamplerParams(Structure):
    _fields_ = [("temperature", c_float), ("top_k", c_int32), ("top_p", c_float), ("min_p", c_float), ("repeat_penalty", c_float),
                ("frequency_penalty", c_float), ("presence_penalty", c_float), ("repeat_last_n", c_int32)]


_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        l = csrc.load(csrc.HOST_LIBRARY)
        l.lgml_host_last_error.restype = c_char_p
        l.lgml_st_open.restype, l.lgml_st_open.argtypes = c_void_p, [c_char_p]
        l.lgml_st_count.restype, l.lgml_st_count.argtypes = c_int, [c_void_p]
        l.lgml_st_get.restype, l.lgml_st_get.argtypes = POINTER(StEntry), [c_void_p, c_int]
        l.lgml_st_close.restype, l.lgml_st_close.argtypes = None, [c_void_p]
        l.lgml_st_read.restype, l.lgml_st_read.argtypes = c_int, [c_char_p, c_int64, c_int64, c_void_p]
        l.lgml_sampler_new.restype, l.lgml_sampler_new.argtypes = c_void_p, [POINTER(SamplerParams), c_uint64]
        l.lgml_sampler_free.restype, l.lgml_sampler_free.argtypes = None, [c_void_p]
        l.lgml_sampler_set_bias.restype, l.lgml_sampler_set_bias.argtypes = c_int, [c_void_p, c_void_p, c_void_p, c_int]
        l.lgml_sampler_accept.restype, l.lgml_sampler_accept.argtypes = c_int, [c_void_p, c_int32]
        l.lgml_sampler_reset.restype, l.lgml_sampler_reset.argtypes = None, [c_void_p]
        l.lgml_sampler_history.restype, l.lgml_sampler_history.argtypes = c_int, [c_void_p, c_void_p, c_int]
        l.lgml_sampler_state.restype, l.lgml_sampler_state.argtypes = None, [c_void_p, c_void_p]
        l.lgml_sampler_next_u64.restype, l.lgml_sampler_next_u64.argtypes = c_uint64, [c_void_p]
        l.lgml_sampler_uniform.restype, l.lgml_sampler_uniform.argtypes = c_double, [c_void_p]
        l.lgml_log_min_p.restype, l.lgml_log_min_p.argtypes = c_float, [c_float]
        l.lgml_sampler_sample.restype, l.lgml_sampler_sample.argtypes = c_int, [c_void_p, c_void_p, c_int, c_void_p]
        l.lgml_sampler_sample_candidates.restype, l.lgml_sampler_sample_candidates.argtypes = c_int, [c_void_p, c_void_p, c_void_p, c_int]
        l.lgml_sampler_logprobs.restype, l.lgml_sampler_logprobs.argtypes = c_int, [c_void_p, c_int32, c_int, POINTER(c_double), c_void_p, c_void_p]
        _lib = l
    return _lib


def last_error() -> str:
    return lib().lgml_host_last_error().decode("utf-8", "replace")
