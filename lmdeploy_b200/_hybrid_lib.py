"""ctypes binding of libb200hybrid.so (include/b200_hybrid.h): the operators of hybrid decoders.  Built on first use from
lmdeploy_b200/csrc/hybrid (one translation unit, seconds with nvcc); there is no fallback when it cannot be built or loaded."""
import ctypes as C
import os

from ._lib import B200LibraryError

BF16, F32 = 1, 2
MAX_TAPS = 16


class Rotary(C.Structure):
    _fields_ = [("freqs", C.c_void_p), ("pairs", C.c_int), ("magnitude", C.c_float)]


class LatentArgs(C.Structure):
    """b200h_latent_args."""
    _fields_ = [
        ("n", C.c_int), ("heads", C.c_int), ("dim", C.c_int), ("rot_dim", C.c_int), ("vdim", C.c_int), ("kv_rank", C.c_int),
        ("q_rank", C.c_int), ("block_len", C.c_int), ("scale", C.c_float), ("eps", C.c_float), ("rot", Rotary),
        ("dq", C.c_void_p), ("ld_dq", C.c_int64), ("dkv", C.c_void_p), ("ld_dkv", C.c_int64),
        ("q_norm", C.c_void_p), ("kv_norm", C.c_void_p), ("cq", C.c_void_p),
        ("q", C.c_void_p), ("ld_q", C.c_int64), ("sink", C.c_void_p),
        ("q_lat", C.c_void_p), ("q_rot", C.c_void_p), ("o_lat", C.c_void_p), ("ml", C.c_void_p), ("splits", C.c_int),
        ("o_heads", C.c_void_p),
        ("tok_seq", C.c_void_p), ("tok_pos", C.c_void_p), ("block_ptrs", C.c_void_p), ("cu_blocks", C.c_void_p),
        ("layer_off", C.c_int64), ("rot_off", C.c_int64), ("dtype", C.c_int), ("stream", C.c_void_p),
    ]


class ExpertArgs(C.Structure):
    """b200h_expert_args."""
    _fields_ = [
        ("n", C.c_int), ("width", C.c_int), ("ff", C.c_int), ("experts", C.c_int), ("top", C.c_int), ("dtype", C.c_int),
        ("x", C.c_void_p), ("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p), ("ids", C.c_void_p), ("wts", C.c_void_p),
        ("out", C.c_void_p), ("mid", C.c_void_p), ("counts", C.c_void_p), ("lists", C.c_void_p), ("stream", C.c_void_p),
        ("act", C.c_int), ("scale_input", C.c_int),
    ]


class WindowArgs(C.Structure):
    """b200h_window_args."""
    _fields_ = [
        ("n", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int), ("dim", C.c_int), ("vdim", C.c_int), ("block_len", C.c_int),
        ("window", C.c_int), ("splits", C.c_int), ("scale", C.c_float), ("softcap", C.c_float), ("eps", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("ld", C.c_int64),
        ("bias", C.c_void_p), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p), ("qn", C.c_void_p),
        ("r1", C.c_void_p), ("r2", C.c_void_p), ("talk", C.c_void_p), ("gate", C.c_void_p), ("ld_gate", C.c_int64),
        ("ml", C.c_void_p), ("o_part", C.c_void_p), ("scores", C.c_void_p), ("score_ld", C.c_int64), ("y", C.c_void_p),
        ("tok_seq", C.c_void_p), ("tok_pos", C.c_void_p), ("block_ptrs", C.c_void_p), ("cu_blocks", C.c_void_p),
        ("layer_off", C.c_int64), ("v_off", C.c_int64), ("dtype", C.c_int), ("stream", C.c_void_p), ("sink", C.c_void_p),
        ("chunk", C.c_int), ("talk_scores", C.c_int), ("gate_heads", C.c_int),
    ]


class ConvPrepArgs(C.Structure):
    """b200h_conv_prep_args."""
    _fields_ = [
        ("n", C.c_int), ("batch", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int), ("dim", C.c_int), ("taps", C.c_int),
        ("block_len", C.c_int), ("eps", C.c_float), ("rot", Rotary),
        ("qk", C.c_void_p), ("ld", C.c_int64), ("conv", C.c_void_p), ("state", C.c_void_p), ("slot_stride", C.c_int64),
        ("qn", C.c_void_p), ("tok_seq", C.c_void_p), ("tok_pos", C.c_void_p), ("cu_q", C.c_void_p), ("seq_slot", C.c_void_p),
        ("block_ptrs", C.c_void_p), ("cu_blocks", C.c_void_p), ("layer_off", C.c_int64), ("v_off", C.c_int64), ("dtype", C.c_int),
        ("stream", C.c_void_p),
    ]


SCORE_FN = {"softmax": 0, "sigmoid": 1}
GATE_ACT = {"sigmoid": 0, "silu": 1}
EXPERT_ACT = {"silu_gate": 0, "relu2": 1}

_lib = None
P, I, L64, F = C.c_void_p, C.c_int, C.c_int64, C.c_float


def load():
    global _lib
    if _lib is not None:
        return _lib
    from . import build
    path = os.environ.get("B200_HYBRID_LIB_PATH") or build.build_hybrid()
    try:
        lib = C.CDLL(path)
    except OSError as e:  # pragma: no cover
        raise B200LibraryError(f"cannot load {path}: {e}") from e
    lib.b200h_last_error.restype = C.c_char_p
    lib.b200h_embed.argtypes = [P, P, F, P, I, I, I, P]
    lib.b200h_causal_conv.argtypes = [P, P, P, L64, P, P, P, P, I, I, I, I, I, P]
    lib.b200h_residual_group_norm.argtypes = [P, P, I, I, P, I, I, I, F, P, I, P]
    lib.b200h_group_norm_rows.argtypes = [P, P, P, I, I, I, F, P, I, P]
    lib.b200h_depth_mix.argtypes = [P, P, L64, P, I, L64, P]
    lib.b200h_latent_prep.argtypes = [C.POINTER(LatentArgs)]
    lib.b200h_latent_attention.argtypes = [C.POINTER(LatentArgs)]
    lib.b200h_rotate_query.argtypes = [C.POINTER(LatentArgs)]
    lib.b200h_head_gate.argtypes = [P, P, L64, I, I, I, P, I, P]
    lib.b200h_decay_attention.argtypes = [P, P, P, L64, P, P, L64, P, P, I, I, I, I, P, I, P]
    lib.b200h_gated_rms.argtypes = [P, P, P, L64, I, I, F, P, I, P]
    lib.b200h_route.argtypes = [P, P, I, I, I, I, P, P, P]
    lib.b200h_experts.argtypes = [C.POINTER(ExpertArgs)]
    lib.b200h_silu_mul.argtypes = [P, P, P, L64, I, P]
    lib.b200h_weighted_scatter.argtypes = [P, P, P, P, I, I, I, P]
    lib.b200h_argmax.argtypes = [P, L64, I, I, P, P]
    lib.b200h_add_rows.argtypes = [P, P, P, I, I, I, I, P]
    lib.b200h_residual_norm.argtypes = [P, P, P, P, I, I, F, P, I, P]
    lib.b200h_relu2.argtypes = [P, L64, I, P]
    lib.b200h_window_prep.argtypes = [C.POINTER(WindowArgs)]
    lib.b200h_window_attention.argtypes = [C.POINTER(WindowArgs)]
    lib.b200h_route_scored.argtypes = [P, I, P, I, I, I, I, I, P, P, P]
    lib.b200h_parallel_residual_norm.argtypes = [P, P, P, I, F, P, P, P, P, I, I, F, P, P, P, I, P]
    lib.b200h_short_conv.argtypes = [P, L64, P, P, I, P, L64, P, P, P, P, I, I, I, I, I, P]
    lib.b200h_ssm_scan.argtypes = [P, P, L64, P, P, P, P, L64, P, P, I, I, I, I, I, I, P, P, I, P]
    lib.b200h_gate_group_norm.argtypes = [P, P, L64, P, I, I, I, F, P, I, P]
    lib.b200h_conv_rope_prep.argtypes = [C.POINTER(ConvPrepArgs)]
    lib.b200h_softcap.argtypes = [P, L64, F, P]
    lib.b200h_scaled_relu2.argtypes = [P, P, I, I, I, P]
    lib.b200h_head_rope_prep.argtypes = [C.POINTER(WindowArgs), C.POINTER(Rotary)]
    lib.b200h_embed_hashed.argtypes = [P, P, P, I, I, I, P, L64, P, P, P, P, P, I, I, I, I, P]
    lib.b200h_branch_residual_norm.argtypes = [P, P, P, P, P, F, P, I, I, P, I, I, F, P, P, I, P]
    lib.b200h_token_shift.argtypes = [P, P, P, I, P, L64, P, P, P, I, I, I, P, P, I, P]
    lib.b200h_channel_decay_scan.argtypes = [P, P, P, L64, P, P, P, P, L64, P, P, I, I, I, I, I, P, P, I, P]
    lib.b200h_group_norm_gate.argtypes = [P, P, P, L64, I, I, I, I, F, P, I, P]
    lib.b200h_xielu.argtypes = [P, L64, P, I, P]
    lib.b200h_tanh.argtypes = [P, L64, I, P]
    lib.b200h_route_grouped.argtypes = [P, I, P, P, I, I, I, I, I, I, I, I, F, P, P, P]
    _lib = lib
    return lib


def check(rc, what=""):
    if rc != 0:
        raise B200LibraryError(f"{what} failed (code {rc}): {load().b200h_last_error().decode()}")
