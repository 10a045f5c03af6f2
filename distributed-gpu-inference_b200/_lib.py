"""ctypes loader for libb200_kv.so — the C-ABI library declared in include/b200_kv.h.

There is no CPU or pure-torch fallback: if the library is missing or does not load, every op raises.
Build it with ``python -c "import __graft_entry__ as g; g.build()"`` or ``make -C <package>/csrc``.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_uint, c_void_p

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libb200_kv.so")

# name -> (restype, argtypes); mirrors include/b200_kv.h one to one
SIGNATURES = {
    "b200_abi_version": (c_int, []),
    "b200_last_error": (c_char_p, []),
    "b200_kv_append": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p],
    ),
    "b200_paged_decode_attn": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
         c_int64, c_float, c_int, c_int, c_void_p, c_size_t, c_int, c_uint, c_void_p],
    ),
    "b200_rope_append_decode_attn": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64, c_float, c_int, c_int, c_void_p, c_size_t,
         c_int, c_uint, c_void_p],
    ),
    "b200_paged_decode_attn_prefix": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
         c_int64, c_float, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_int, c_uint, c_void_p],
    ),
    "b200_rope_append_decode_attn_prefix": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64, c_float, c_int, c_int, c_int, c_int,
         c_void_p, c_size_t, c_int, c_uint, c_void_p],
    ),
    "b200_paged_decode_attn_prefix_plan": (
        c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int)]),
    "b200_paged_decode_attn_static": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
         c_int64, c_float, c_int, c_int, c_int, c_uint, c_void_p],
    ),
    "b200_paged_decode_attn_workspace": (c_size_t, [c_int, c_int, c_int, c_int]),
    "b200_paged_decode_attn_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "b200_kv_pack_layers_wire": (
        c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_void_p]),
    "b200_kv_unpack_layers_wire": (
        c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_void_p]),
    "b200_kv_move_blocks_layers": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64,
         c_int, c_void_p],
    ),
    "b200_add_rmsnorm": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int64, c_int64, c_int, c_void_p]),
    "b200_rope_kv_append": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
         c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p],
    ),
    "b200_rope_kv_append_prompt": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
         c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p],
    ),
    "b200_argmax_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "b200_argmax_rows_keys": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "b200_argmax_keys_decode": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "b200_silu_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64, c_int, c_void_p]),
    "b200_kv_gather_dense": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_int,
         c_void_p],
    ),
    "b200_kv_pack": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p]),
    "b200_kv_unpack": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p]),
    "b200_kv_pack_layers": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p],
    ),
    "b200_kv_unpack_layers": (
        c_int,
        [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p],
    ),
}

# libb200_mixers.so (include/b200_mixers.h): ragged-batch mixers and feed-forward pieces
MIXER_LIB_PATH = os.path.join(_PKG_DIR, "libb200_mixers.so")
MIXER_SIGNATURES = {
    "b200_mixers_abi_version": (c_int, []),
    "b200_mixers_last_error": (c_char_p, []),
    "b200_offset_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p]),
    "b200_postnorm_residual": (
        c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_float, c_void_p, c_void_p, c_float, c_int, c_int, c_int,
                c_void_p]),
    "b200_value_prep_append": (
        c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p, c_void_p,
                c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p]),
    "b200_biased_attn_tile_tokens": (c_int, [c_int, c_int, c_int]),
    "b200_biased_paged_attn": (
        c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                c_void_p]),
    "b200_biased_prompt_attn_supported": (c_int, [c_int, c_int, c_int]),
    "b200_biased_prompt_attn_tile_tokens": (c_int, [c_int, c_int]),
    "b200_biased_prompt_attn": (
        c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                c_void_p]),
    "b200_gated_scan": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                c_int, c_int, c_int, c_int, c_void_p]),
    "b200_head_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int64, c_int, c_int, c_void_p]),
    "b200_polynorm": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_float, c_int, c_int, c_int, c_void_p]),
    "b200_sigmoid_topk": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200_scaled_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "b200_grouped_linear_supported": (c_int, [c_int, c_int]),
    "b200_grouped_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_clamped_glu": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_float, c_float, c_int, c_void_p]),
    "b200_expert_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    # pieces for hybrid designs (csrc/b200_hybrid_ops.cu)
    "b200_rms_norm": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_float, c_float, c_int, c_int, c_int,
                              c_void_p]),
    "b200_residual_add2_norm": (
        c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_float, c_void_p, c_float, c_int, c_int, c_int,
                c_void_p]),
    "b200_xielu": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200_rotary_kv_append": (
        c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int64, c_void_p, c_int, c_void_p]),
    "b200_norm_append": (
        c_int, [c_void_p, c_int64, c_void_p, c_float, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200_mixed_paged_attn": (
        c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_int, c_int, c_float,
                c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_mixed_prompt_attn_supported": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "b200_mixed_prompt_attn_splits": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "b200_mixed_prompt_attn_workspace": (c_size_t, [c_int, c_int, c_int, c_int]),
    "b200_mixed_prompt_attn": (
        c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_void_p, c_int,
                c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "b200_causal_conv_silu": (
        c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                c_void_p]),
    "b200_delta_scan": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p]),
    "b200_head_rmsnorm_gated": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_int64, c_int, c_int, c_int, c_void_p]),
    # side-by-side mixers, post-norm sublayers, grouped softmax routing (csrc/b200_parallel_ops.cu)
    "b200_qknorm_rotary_append": (
        c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_float, c_void_p, c_int,
                c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_int,
                c_void_p]),
    "b200_retention_scan": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                c_int, c_int, c_int, c_void_p]),
    "b200_retention_carry": (
        c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200_retention_apply_carry": (
        c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_head_norm_act_gate": (
        c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_float, c_int64, c_int, c_int,
                c_int, c_void_p]),
    "b200_branch_postnorm_residual": (
        c_int, [c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p, c_int64, c_float, c_void_p, c_void_p, c_void_p,
                c_float, c_int, c_int, c_int, c_void_p]),
    "b200_cast_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "b200_softmax_group_topk": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_gather_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "b200_weighted_expert_combine": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                c_void_p]),
    # chunked masks, values inside wider rows, several score maps per value head (csrc/b200_hybrid_ops.cu)
    "b200_mixed_paged_attn_ext": (
        c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_int, c_int, c_int,
                c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_mixed_prompt_attn_ext": (
        c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_int,
                c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                c_void_p]),
    "b200_qknorm_rotary_append_ext": (
        c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int,
                c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_int,
                c_void_p]),
    # token shift, gated post-norm sublayers, a decoupled rotated key part (csrc/b200_gated_ops.cu)
    "b200_token_shift": (
        c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_latent_rotary_append": (
        c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_float, c_void_p,
                c_float, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_head_diff_norm": (
        c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int, c_float, c_float, c_float, c_int64, c_int, c_int, c_int,
                c_int, c_void_p]),
    "b200_gated_postnorm_residual": (
        c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p, c_float, c_void_p, c_float, c_int, c_int,
                c_int, c_void_p]),
    "b200_relu_squared": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p]),
    "b200_router_logits": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "b200_gated_table_rows": (
        c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_int, c_void_p]),
}

_lock = threading.Lock()
_lib = None
_mixers = None


class B200LibraryError(RuntimeError):
    """The CUDA extension is missing, failed to load, or an entry point reported an error."""


def load() -> ctypes.CDLL:
    """Load (once) and return the library with argument types set.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise B200LibraryError(
                f"{LIB_PATH} not found: the sm_100a extension is not built (run __graft_entry__.build()). "
                "There is no CPU fallback for the paged-KV ops."
            )
        try:
            lib = ctypes.CDLL(LIB_PATH)
        except OSError as exc:
            raise B200LibraryError(f"cannot load {LIB_PATH}: {exc}") from exc
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means header and library drifted apart
            fn.restype = restype
            fn.argtypes = argtypes
        if lib.b200_abi_version() != 1:
            raise B200LibraryError(f"ABI version {lib.b200_abi_version()} != 1")
        _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().b200_last_error()
        raise B200LibraryError(f"{what} failed (code {rc}): {msg.decode() if msg else ''}")


def _build_mixers() -> None:
    """Compile libb200_mixers.so in-tree (its sources in parallel, under a minute).  A checkout without built files compiles it
    at first use; concurrent callers are serialised by a lock file and the library appears atomically."""
    import fcntl
    import subprocess

    csrc = os.path.join(_PKG_DIR, "csrc")
    with open(os.path.join(csrc, ".mixers.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if os.path.exists(MIXER_LIB_PATH):
            return
        proc = subprocess.run(["make", "-j4", "-C", csrc, "mixers"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
        if proc.returncode != 0 or not os.path.exists(MIXER_LIB_PATH):
            raise B200LibraryError("building libb200_mixers.so failed:\n" + proc.stdout.decode(errors="replace")[-4000:])


def load_mixers() -> ctypes.CDLL:
    """Load (once) libb200_mixers.so, building it first when the checkout has no built copy.  No CPU fallback."""
    global _mixers
    if _mixers is not None:
        return _mixers
    with _lock:
        if _mixers is not None:
            return _mixers
        if not os.path.exists(MIXER_LIB_PATH):
            _build_mixers()
        try:
            lib = ctypes.CDLL(MIXER_LIB_PATH)
        except OSError as exc:
            raise B200LibraryError(f"cannot load {MIXER_LIB_PATH}: {exc}") from exc
        for name, (restype, argtypes) in MIXER_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        if lib.b200_mixers_abi_version() != 1:
            raise B200LibraryError(f"mixers ABI version {lib.b200_mixers_abi_version()} != 1")
        _mixers = lib
    return _mixers


def check_mixers(rc: int, what: str) -> None:
    if rc != 0:
        msg = load_mixers().b200_mixers_last_error()
        raise B200LibraryError(f"{what} failed (code {rc}): {msg.decode() if msg else ''}")
