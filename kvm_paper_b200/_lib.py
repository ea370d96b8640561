"""ctypes binding of libkvm_b200.so (declarations mirror include/kvm_b200.h).

The library is the only compute path of this package: importing this module without the built
library raises, there is no fallback.
"""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkvm_b200.so")

KVM_OK = 0
PREFILL_CHAIN, PREFILL_ATTENTION, PREFILL_LEGACY_ATTENTION, PREFILL_LEGACY_CHAIN = 1, 2, 4, 8
PREFILL_TEST_WITHHOLD_ARRIVAL = 16
PREFILL_KEYS_PREPARED = 32
ERROR_NAMES = {1: "bad argument", 2: "capacity", 3: "device timeout", 4: "CUDA error", 5: "unsupported"}


class KvmLayer(C.Structure):
    _fields_ = [
        ("n_q_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("chunk_len", C.c_int32), ("n_bswa_chunks", C.c_int32), ("rope_dim", C.c_int32),
        ("sink_len", C.c_int32), ("gate_keys", C.c_int32), ("gate_values", C.c_int32),
        ("gate_appends", C.c_int32), ("gate_initial", C.c_int32), ("ln_eps", C.c_float),
        ("ln_weight_dev", C.c_void_p), ("ln_bias_dev", C.c_void_p),
        ("front_temp_dev", C.c_void_p), ("state_temp_dev", C.c_void_p),
    ]


class KvmTensor4(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_t", C.c_int64)]


class KvmMemory(C.Structure):
    _fields_ = [("k_sum", C.c_void_p), ("v_sum", C.c_void_p), ("vlen", C.c_void_p),
                ("k_attn", C.c_void_p), ("v_attn", C.c_void_p), ("capacity", C.c_int32)]


class KvmUpdatePlan(C.Structure):
    _fields_ = [("state_before", C.c_int32), ("n_append", C.c_int32), ("version_row", C.c_int32),
                ("reserved", C.c_int32)]


class KvmPrefillLayout(C.Structure):
    _fields_ = [("status_offset", C.c_size_t), ("pool_k_offset", C.c_size_t), ("pool_v_offset", C.c_size_t),
                ("version_table_offset", C.c_size_t), ("prepared_keys_offset", C.c_size_t),
                ("gated_keys_offset", C.c_size_t), ("pool_rows", C.c_int64), ("total_bytes", C.c_size_t)]


class KvmPrologue(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("q_lin", "k_lin", "v_lin", "gate_lin", "shift_q", "shift_k", "shift_v",
                                          "prev_q", "prev_k", "prev_v", "ln_q_w", "ln_q_b", "ln_k_w", "ln_k_b")] + [
        ("ln_qk_eps", C.c_float), ("cos", C.c_void_p), ("sin", C.c_void_p), ("rope_stride_b", C.c_int64)]


class KvmDecodeCache(C.Structure):
    _fields_ = [("memory", KvmMemory), ("ring_k", C.c_void_p), ("ring_v", C.c_void_p),
                ("ring_gate", C.c_void_p), ("total_len", C.c_void_p), ("state_len", C.c_void_p)]


EXPORTS = [
    "kvm_prefill_workspace_bytes", "kvm_prefill_forward", "kvm_decode_workspace_bytes", "kvm_decode_step",
    "kvm_memory_refresh", "kvm_last_error_string", "kvm_abi_version", "kvm_decode_step_static", "kvm_prefill_status", "kvm_decode_run",
    "kvm_decode_status", "kvm_prefill_workspace_layout", "kvm_interleave_shards", "kvm_prologue_forward",
    "kvm_prefill_forward_gathered",
]
STATIC_SCRATCH_BYTES = 32 << 20

_lib = None


def load():
    """Load the library (once) and declare the signatures.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m kvm_paper_b200.build` "
            "(this package has no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    LP = C.POINTER
    lib.kvm_prefill_workspace_bytes.restype = C.c_size_t
    lib.kvm_prefill_workspace_bytes.argtypes = [LP(KvmLayer), C.c_int32, C.c_int64, C.c_int64]
    lib.kvm_prefill_forward.restype = C.c_int
    lib.kvm_prefill_forward.argtypes = [
        LP(KvmLayer), C.c_int32, C.c_int64, KvmTensor4, KvmTensor4, KvmTensor4, KvmTensor4,
        C.c_void_p, LP(KvmUpdatePlan), C.c_int32, C.c_int64, KvmMemory, C.c_void_p, C.c_void_p,
        C.c_void_p, C.c_size_t, C.c_uint32, C.c_void_p]
    lib.kvm_prefill_forward_gathered.restype = C.c_int
    lib.kvm_prefill_forward_gathered.argtypes = [
        LP(KvmLayer), C.c_int32, C.c_int64, KvmTensor4, KvmTensor4, KvmTensor4, KvmTensor4,
        C.c_void_p, LP(KvmUpdatePlan), C.c_int32, C.c_int64, KvmMemory, C.c_int32, C.c_int32, LP(C.c_void_p), C.c_void_p,
        C.c_void_p, C.c_size_t, C.c_uint32, C.c_void_p]
    lib.kvm_prefill_status.restype = C.c_int
    lib.kvm_prefill_status.argtypes = [C.c_void_p, C.c_void_p]
    lib.kvm_prefill_workspace_layout.restype = C.c_int
    lib.kvm_prefill_workspace_layout.argtypes = [LP(KvmLayer), C.c_int32, C.c_int64, C.c_int64, LP(KvmPrefillLayout)]
    lib.kvm_decode_status.restype = C.c_int
    lib.kvm_decode_status.argtypes = [LP(KvmLayer), C.c_int32, C.c_void_p, C.c_void_p]
    lib.kvm_decode_workspace_bytes.restype = C.c_size_t
    lib.kvm_decode_workspace_bytes.argtypes = [LP(KvmLayer), C.c_int32, C.c_int32]
    lib.kvm_decode_step.restype = C.c_int
    lib.kvm_decode_step.argtypes = [
        LP(KvmLayer), C.c_int32, KvmDecodeCache, KvmTensor4, KvmTensor4, KvmTensor4, KvmTensor4,
        C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.kvm_decode_run.restype = C.c_int
    lib.kvm_decode_run.argtypes = [
        LP(KvmLayer), C.c_int32, KvmDecodeCache, C.c_int32, KvmTensor4, KvmTensor4, KvmTensor4, KvmTensor4,
        C.c_int64, C.c_int64, C.c_int64, C.c_void_p, LP(C.c_int32), LP(C.c_int32), C.c_void_p, C.c_void_p,
        C.c_size_t, C.c_void_p]
    # decode step with the scratch inside the library (for callers that cannot allocate device memory)
    lib.kvm_decode_step_static.restype = C.c_int
    lib.kvm_decode_step_static.argtypes = [
        LP(KvmLayer), C.c_int32, KvmDecodeCache, KvmTensor4, KvmTensor4, KvmTensor4, KvmTensor4,
        C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.kvm_memory_refresh.restype = C.c_int
    lib.kvm_memory_refresh.argtypes = [LP(KvmLayer), C.c_int32, KvmMemory, C.c_void_p, C.c_void_p]
    lib.kvm_prologue_forward.restype = C.c_int
    lib.kvm_prologue_forward.argtypes = [LP(KvmLayer), C.c_int32, C.c_int64, LP(KvmPrologue), C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_int64, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.kvm_interleave_shards.restype = C.c_int
    lib.kvm_interleave_shards.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_void_p]
    lib.kvm_last_error_string.restype = C.c_char_p
    lib.kvm_last_error_string.argtypes = []
    lib.kvm_abi_version.restype = C.c_int
    lib.kvm_abi_version.argtypes = []
    _lib = lib
    return lib


class KvmError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"kvm_b200 status {code} ({ERROR_NAMES.get(code, '?')}): {message}")
        self.code = code


def check(code: int) -> None:
    """Map a status code to the exception type the reference would raise for the same misuse:
    ValueError for unsupported/bad arguments, RuntimeError otherwise."""
    if code == KVM_OK:
        return
    msg = load().kvm_last_error_string().decode()
    if code in (1, 5):
        raise ValueError(f"kvm_b200 status {code} ({ERROR_NAMES[code]}): {msg}")
    raise KvmError(code, msg)
