"""ctypes loader for the CPU oracle.  TEST INFRASTRUCTURE ONLY.

The oracle is the checker: tests, the smoke entry and the benchmark's CPU-baseline leg call
it; the product library never imports, links or executes it.  Arrays are numpy: bf16 tensors
travel as uint16 bit patterns, F32 and I32 as themselves.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_float, c_int, c_int32, c_int64, c_size_t, c_uint16, c_uint32, c_uint64

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libloom_oracle.so")

HEAD_DIM = 128
PAGE_SIZE = 16
STATE_WIDTH = 130

# Same order as ContractError (crates/loom-infer/src/error.rs:6-109).
STATUS_NAMES = [
    "Ok", "ZeroDimension", "ElementCountOverflow", "InvalidEpsilon", "UnsupportedHeadDimension",
    "UnsupportedPageSize", "InvalidHeadMapping", "InvalidPartitionCount", "InvalidIndptrStart",
    "NonMonotonicIndptr", "EmptyRaggedRequest", "RaggedQueryLongerThanKv",
    "InvalidPageIndptrStart", "NonMonotonicPageIndptr", "EmptyPagedRequest",
    "PageIndexOutOfRange", "InvalidLastPageLength", "InvalidRotaryDimension", "InvalidRopeScale",
    "InvalidRopeTheta", "NegativePositionId", "UnsupportedAppendTokenCount",
    "AppendBatchIndexOutOfRange", "AppendPositionOutOfRange", "DuplicatePageAppendSlot",
    "DuplicatePageAppendTokenSlot", "UnsupportedDType", "LengthMismatch",
]


class _Error(ctypes.Structure):
    _fields_ = [("code", c_int32), ("buffer", ctypes.c_char * 24), ("a", c_int64),
                ("b", c_int64), ("c", c_int64), ("d", c_int64)]


class _Spec(ctypes.Structure):
    _fields_ = [("batch_size", c_size_t), ("max_num_pages", c_size_t),
                ("num_query_heads", c_size_t), ("num_kv_heads", c_size_t)]


class OracleError(Exception):
    """A ContractError reported by the oracle: variant name plus its payload."""

    def __init__(self, err: _Error):
        self.variant = STATUS_NAMES[err.code]
        self.buffer = err.buffer.decode()
        self.payload = (err.a, err.b, err.c, err.d)
        super().__init__(f"{self.variant} buffer={self.buffer!r} payload={self.payload}")


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc -O2 -ffp-contract=off)."""
    source = os.path.join(_HERE, "loom_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)
             or os.path.getmtime(_LIB_PATH) < os.path.getmtime(source))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libloom_oracle.so"], check=True,
                       capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.lo_digest_u16.restype = c_uint64
        _lib.lo_digest_u32.restype = c_uint64
        _lib.lo_bf16_from_f32.restype = c_uint16
        _lib.lo_bf16_from_f32.argtypes = [c_float]
        _lib.lo_bf16_to_f32.restype = c_float
        _lib.lo_bf16_to_f32.argtypes = [c_uint16]
    return _lib


def _u16(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return a, a.ctypes.data_as(POINTER(c_uint16)), c_size_t(a.size)


def _i32(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(POINTER(c_int32)), c_size_t(a.size)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(POINTER(c_float)), c_size_t(a.size)


def _check(rc, err):
    if rc != 0:
        raise OracleError(err)


# ---- bf16 / fixture / digests ----------------------------------------------------------------

def bf16_from_f32(values) -> np.ndarray:
    """Round-to-nearest-even F32 -> bf16 bit patterns (NaN quieted), vectorised."""
    x = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    nan = (x & 0x7FFFFFFF) > 0x7F800000
    rounded = ((x >> 16) + (((x & 0x8000) != 0) & ((x & 0x17FFF) != 0))).astype(np.uint16)
    return np.where(nan, ((x >> 16) | 0x40).astype(np.uint16), rounded)


def bf16_to_f32(bits) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def fixture_bf16(length: int, salt: int) -> np.ndarray:
    """deterministic_bf16 (crates/loom-infer-validation/src/support/fixture.rs:5-16)."""
    out = np.empty(length, dtype=np.uint16)
    lib().lo_fixture_bf16(out.ctypes.data_as(POINTER(c_uint16)), c_size_t(length), c_uint64(salt))
    return out


def digest_bf16(bits) -> int:
    a, p, n = _u16(bits)
    return lib().lo_digest_u16(p, n)


def digest_f32(values) -> int:
    a = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    return lib().lo_digest_u32(a.ctypes.data_as(POINTER(c_uint32)), c_size_t(a.size))


def digest_i32(values) -> int:
    a = np.ascontiguousarray(values, dtype=np.int32).view(np.uint32)
    return lib().lo_digest_u32(a.ctypes.data_as(POINTER(c_uint32)), c_size_t(a.size))


# ---- spec + metadata -------------------------------------------------------------------------

def paged_spec(batch, max_pages, qh, kvh, head_dim=HEAD_DIM, page_size=PAGE_SIZE) -> _Spec:
    spec, err = _Spec(), _Error()
    _check(lib().lo_paged_spec_new(c_size_t(batch), c_size_t(max_pages), c_size_t(qh),
                                   c_size_t(kvh), c_size_t(head_dim), c_size_t(page_size),
                                   ctypes.byref(spec), ctypes.byref(err)), err)
    return spec


def validate_page_table(spec, indptr, indices, last):
    err = _Error()
    _, ip, il = _i32(indptr)
    _, xp, xl = _i32(indices)
    _, lp, ll = _i32(last)
    _check(lib().lo_validate_page_table(ctypes.byref(spec), ip, il, xp, xl, lp, ll,
                                        ctypes.byref(err)), err)


def append_validate_page_table(spec, indptr, indices, last):
    err = _Error()
    _, ip, il = _i32(indptr)
    _, xp, xl = _i32(indices)
    _, lp, ll = _i32(last)
    _check(lib().lo_append_validate_page_table(ctypes.byref(spec), ip, il, xp, xl, lp, ll,
                                               ctypes.byref(err)), err)


def append_tokens_validate(spec, tokens, batch_indices, positions, indptr, indices, last,
                           max_tokens=64):
    """Returns the (page, offset) slot of every token, or raises OracleError."""
    err = _Error()
    _, bp, bl = _i32(batch_indices)
    _, pp, pl = _i32(positions)
    _, ip, il = _i32(indptr)
    _, xp, xl = _i32(indices)
    _, lp, ll = _i32(last)
    slots = np.zeros((max(tokens, 1), 2), dtype=np.int64)
    _check(lib().lo_append_tokens_validate(ctypes.byref(spec), c_size_t(tokens),
                                           c_size_t(max_tokens), bp, bl, pp, pl, ip, il, xp, xl,
                                           lp, ll, slots.ctypes.data_as(POINTER(c_int64)),
                                           ctypes.byref(err)), err)
    return [tuple(int(v) for v in row) for row in slots[:tokens]]


def request_kv_lens(indptr, last) -> np.ndarray:
    indptr = np.asarray(indptr, dtype=np.int64)
    return (indptr[1:] - indptr[:-1] - 1) * PAGE_SIZE + np.asarray(last, dtype=np.int64)


# ---- references ------------------------------------------------------------------------------

def paged_decode(spec, q, k_pages, v_pages, indptr, indices, last, threads=1, out=None, lse=None):
    """paged_batch_decode_bf16_reference; returns (O bf16 bits, LSE f32)."""
    err = _Error()
    q, qp, ql = _u16(q)
    k, kp, kl = _u16(k_pages)
    v, vp, vl = _u16(v_pages)
    _, ip, il = _i32(indptr)
    _, xp, xl = _i32(indices)
    _, lp, ll = _i32(last)
    if out is None:
        out = np.full(spec.batch_size * spec.num_query_heads * HEAD_DIM, 0x7FC0, dtype=np.uint16)
    if lse is None:
        lse = np.full(spec.batch_size * spec.num_query_heads, np.nan, dtype=np.float32)
    _check(lib().lo_paged_decode_ref(ctypes.byref(spec), qp, ql, kp, kl, vp, vl, ip, il, xp, xl,
                                     lp, ll, out.ctypes.data_as(POINTER(c_uint16)),
                                     c_size_t(out.size), lse.ctypes.data_as(POINTER(c_float)),
                                     c_size_t(lse.size), c_int(threads), ctypes.byref(err)), err)
    return out, lse


def single_decode(kv_len, qh, kvh, q, k, v):
    err = _Error()
    _, qp, _n = _u16(q)
    _, kp, _n = _u16(k)
    _, vp, _n = _u16(v)
    out = np.zeros(qh * HEAD_DIM, dtype=np.uint16)
    lse = np.zeros(qh, dtype=np.float32)
    _check(lib().lo_single_decode_ref(c_size_t(kv_len), c_size_t(qh), c_size_t(kvh), qp, kp, vp,
                                      out.ctypes.data_as(POINTER(c_uint16)),
                                      lse.ctypes.data_as(POINTER(c_float)), ctypes.byref(err)), err)
    return out, lse


def split_k_partition_range(kv_len, partitions, partition):
    start, end = c_size_t(), c_size_t()
    if lib().lo_split_k_partition_range(c_size_t(kv_len), c_size_t(partitions),
                                        c_size_t(partition), ctypes.byref(start),
                                        ctypes.byref(end)):
        return None
    return start.value, end.value


def split_k_partials(kv_len, qh, kvh, partitions, q, k, v, workspace=None):
    err = _Error()
    _, qp, _n = _u16(q)
    _, kp, _n = _u16(k)
    _, vp, _n = _u16(v)
    if workspace is None:
        workspace = np.full(qh * partitions * STATE_WIDTH, np.nan, dtype=np.float32)
    _check(lib().lo_split_k_partials_ref(c_size_t(kv_len), c_size_t(qh), c_size_t(kvh),
                                         c_size_t(partitions), qp, kp, vp,
                                         workspace.ctypes.data_as(POINTER(c_float)),
                                         c_size_t(workspace.size), ctypes.byref(err)), err)
    return workspace


def split_k_merge(qh, partitions, workspace):
    err = _Error()
    w, wp, wl = _f32(workspace)
    out = np.zeros(qh * HEAD_DIM, dtype=np.uint16)
    lse = np.zeros(qh, dtype=np.float32)
    _check(lib().lo_split_k_merge_ref(c_size_t(qh), c_size_t(partitions), wp, wl,
                                      out.ctypes.data_as(POINTER(c_uint16)),
                                      lse.ctypes.data_as(POINTER(c_float)), ctypes.byref(err)), err)
    return out, lse


def paged_split_k(spec, partitions, q, k_pages, v_pages, indptr, indices, last):
    """Paged split-K: page-balanced partials then LSE merge.  Returns (O, LSE, workspace)."""
    err = _Error()
    _, qp, _n = _u16(q)
    _, kp, _n = _u16(k_pages)
    _, vp, _n = _u16(v_pages)
    _, ip, _n = _i32(indptr)
    _, xp, xl = _i32(indices)
    _, lp, _n = _i32(last)
    states = spec.batch_size * spec.num_query_heads
    workspace = np.full(states * partitions * STATE_WIDTH, np.nan, dtype=np.float32)
    _check(lib().lo_paged_split_k_partials_ref(ctypes.byref(spec), c_size_t(partitions), qp, kp,
                                               vp, ip, xp, xl, lp,
                                               workspace.ctypes.data_as(POINTER(c_float)),
                                               ctypes.byref(err)), err)
    out = np.zeros(states * HEAD_DIM, dtype=np.uint16)
    lse = np.zeros(states, dtype=np.float32)
    lib().lo_paged_split_k_merge_ref(ctypes.byref(spec), c_size_t(partitions),
                                     workspace.ctypes.data_as(POINTER(c_float)),
                                     out.ctypes.data_as(POINTER(c_uint16)),
                                     lse.ctypes.data_as(POINTER(c_float)))
    return out, lse, workspace


def rope(tokens, qh, kh, q, k, positions, head_dim=HEAD_DIM, rotary_dim=HEAD_DIM, scale=1.0,
         theta=10000.0):
    err = _Error()
    _, qp, ql = _u16(q)
    _, kp, kl = _u16(k)
    _, pp, pl = _i32(positions)
    q_out = np.full(tokens * qh * head_dim, 0x7FC0, dtype=np.uint16)
    k_out = np.full(tokens * kh * head_dim, 0x7FC0, dtype=np.uint16)
    _check(lib().lo_rope_ref(c_size_t(tokens), c_size_t(qh), c_size_t(kh), c_size_t(head_dim),
                             c_size_t(rotary_dim), c_float(scale), c_float(theta), qp, ql, kp, kl,
                             pp, pl, q_out.ctypes.data_as(POINTER(c_uint16)), c_size_t(q_out.size),
                             k_out.ctypes.data_as(POINTER(c_uint16)), c_size_t(k_out.size),
                             ctypes.byref(err)), err)
    return q_out, k_out


def rope_append(spec, q, k, v, indptr, indices, last, k_pages, v_pages):
    """rope_paged_kv_append_bf16_reference.  Returns (Q out, K pages, V pages) copies."""
    err = _Error()
    _, qp, ql = _u16(q)
    _, kp, kl = _u16(k)
    _, vp, vl = _u16(v)
    _, ip, il = _i32(indptr)
    _, xp, xl = _i32(indices)
    _, lp, ll = _i32(last)
    q_out = np.full(spec.batch_size * spec.num_query_heads * HEAD_DIM, 0x7FC0, dtype=np.uint16)
    kpg = np.array(k_pages, dtype=np.uint16, copy=True)
    vpg = np.array(v_pages, dtype=np.uint16, copy=True)
    _check(lib().lo_rope_append_ref(ctypes.byref(spec), qp, ql, kp, kl, vp, vl, ip, il, xp, xl,
                                    lp, ll, q_out.ctypes.data_as(POINTER(c_uint16)),
                                    c_size_t(q_out.size), kpg.ctypes.data_as(POINTER(c_uint16)),
                                    c_size_t(kpg.size), vpg.ctypes.data_as(POINTER(c_uint16)),
                                    c_size_t(vpg.size), ctypes.byref(err)), err)
    return q_out, kpg, vpg


def rope_append_tokens(spec, tokens, q, k, v, batch_indices, positions, indptr, indices, last,
                       k_pages, v_pages, max_tokens=64):
    """rope_paged_kv_append_tokens_bf16_reference (max_tokens=0 lifts the 64-token cap)."""
    err = _Error()
    _, qp, ql = _u16(q)
    _, kp, kl = _u16(k)
    _, vp, vl = _u16(v)
    _, bp, bl = _i32(batch_indices)
    _, pp, pl = _i32(positions)
    _, ip, il = _i32(indptr)
    _, xp, xl = _i32(indices)
    _, lp, ll = _i32(last)
    q_out = np.full(tokens * spec.num_query_heads * HEAD_DIM, 0x7FC0, dtype=np.uint16)
    kpg = np.array(k_pages, dtype=np.uint16, copy=True)
    vpg = np.array(v_pages, dtype=np.uint16, copy=True)
    _check(lib().lo_rope_append_tokens_ref(ctypes.byref(spec), c_size_t(tokens),
                                           c_size_t(max_tokens), qp, ql, kp, kl, vp, vl, bp, bl,
                                           pp, pl, ip, il, xp, xl, lp, ll,
                                           q_out.ctypes.data_as(POINTER(c_uint16)),
                                           c_size_t(q_out.size),
                                           kpg.ctypes.data_as(POINTER(c_uint16)),
                                           c_size_t(kpg.size),
                                           vpg.ctypes.data_as(POINTER(c_uint16)),
                                           c_size_t(vpg.size), ctypes.byref(err)), err)
    return q_out, kpg, vpg


# ---- paged causal prefill --------------------------------------------------------------------

class _PrefillSpec(ctypes.Structure):
    _fields_ = [("batch_size", c_size_t), ("nnz_qo", c_size_t), ("max_num_pages", c_size_t),
                ("num_query_heads", c_size_t), ("num_kv_heads", c_size_t)]


def prefill_spec(batch, nnz_qo, max_pages, qh, kvh, head_dim=HEAD_DIM,
                 page_size=PAGE_SIZE) -> _PrefillSpec:
    """Bf16PagedPrefillSpec::new (paged_prefill/mod.rs:29-91)."""
    spec, err = _PrefillSpec(), _Error()
    _check(lib().lo_prefill_spec_new(c_size_t(batch), c_size_t(nnz_qo), c_size_t(max_pages),
                                     c_size_t(qh), c_size_t(kvh), c_size_t(head_dim),
                                     c_size_t(page_size), ctypes.byref(spec), ctypes.byref(err)),
           err)
    return spec


def prefill_validate_metadata(spec, qo_indptr, page_indptr, indices, last):
    err = _Error()
    _, qp, ql = _i32(qo_indptr)
    _, ip, il = _i32(page_indptr)
    _, xp, xl = _i32(indices)
    _, lp, ll = _i32(last)
    _check(lib().lo_prefill_validate_metadata(ctypes.byref(spec), qp, ql, ip, il, xp, xl, lp, ll,
                                              ctypes.byref(err)), err)


def paged_prefill(spec, q, k_pages, v_pages, qo_indptr, page_indptr, indices, last, threads=1):
    """paged_prefill_bf16_reference; returns (O bf16 bits, LSE f32 in the log2 domain)."""
    err = _Error()
    q, qp, ql = _u16(q)
    k, kp, kl = _u16(k_pages)
    v, vp, vl = _u16(v_pages)
    _, op, ol = _i32(qo_indptr)
    _, ip, il = _i32(page_indptr)
    _, xp, xl = _i32(indices)
    _, lp, ll = _i32(last)
    out = np.full(spec.nnz_qo * spec.num_query_heads * HEAD_DIM, 0x7FC0, dtype=np.uint16)
    lse = np.full(spec.nnz_qo * spec.num_query_heads, np.nan, dtype=np.float32)
    _check(lib().lo_paged_prefill_ref(ctypes.byref(spec), qp, ql, kp, kl, vp, vl, op, ol, ip, il,
                                      xp, xl, lp, ll, out.ctypes.data_as(POINTER(c_uint16)),
                                      c_size_t(out.size), lse.ctypes.data_as(POINTER(c_float)),
                                      c_size_t(lse.size), c_int(threads), ctypes.byref(err)), err)
    return out, lse
