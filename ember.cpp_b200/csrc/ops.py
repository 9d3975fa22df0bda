"""The kernels as the parts call them.

`CudaOps` is the only implementation the library ships: it loads the shared library that
build.py makes from this folder's CUDA sources and calls its C entry points on torch's current
stream with raw device pointers.  There is no CPU path and no fallback to library model code; a
missing compiler, a failed build or a missing GPU is an error at construction.

Which kernel runs is decided here from the element types and the shape of the step:
float32 operands take the float32 kernels (FFMA product in a fixed order, plain attention),
bfloat16 operands take the tensor-core kernels.
"""
from __future__ import annotations

import ctypes

import torch

from . import build

_F32, _BF16 = 0, 1
_ACT = {None: 0, "gelu_tanh": 1, "gelu_erf": 2, "relu2": 3}
_LT_WORKSPACE = 32 << 20

_c_int, _c_float, _c_void, _c_size, _c_u64 = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint64

_SIGNATURES = {
    "ember_token_shift": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void],
    "ember_cast_rows": [_c_void, _c_void, _c_size, _c_int, _c_void],
    "ember_table_gate": [_c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_low_rank_out": [_c_void, ctypes.c_longlong, _c_int, _c_int, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int,
                           _c_void],
    "ember_gla_scan": [_c_void, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_void, _c_float, _c_void, _c_void, _c_void, _c_void,
                       _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_int, _c_void],
    "ember_generalized_delta_rule": [_c_void, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_float,
                                     _c_float, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void,
                                     _c_int, _c_void],
    "ember_moe_pick": [_c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void, _c_void, _c_void],
    "ember_moe_combine": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_int, _c_int, _c_int, _c_void],
    "ember_moe_gate_up_act": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int,
                              _c_int, _c_int, _c_float, _c_float, _c_float, _c_void],
    "ember_conv_act": [_c_void, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void,
                       _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_rotate_pairs": [_c_void, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_void, ctypes.c_longlong, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_int, _c_void, _c_void, _c_float, _c_int, _c_int, _c_void],
    "ember_attention_plain_chunked": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int,
                                      _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_void,
                                      _c_int, _c_void],
    "ember_attention_prefill_chunked": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void, _c_void,
                                        _c_int, _c_void, _c_void],
    "ember_attention_decode_chunked": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int,
                                       _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int,
                                       _c_void, _c_void],
    "ember_embed": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_int, _c_float,
                    _c_void],
    "ember_layernorm": [_c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_float, _c_int, _c_void],
    "ember_gather_rows": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_void],
    "ember_take_tokens": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void],
    "ember_act_inplace": [_c_void, _c_size, _c_int, _c_int, _c_void],
    "ember_scale_cap_inplace": [_c_void, _c_size, _c_float, _c_float, _c_void],
    "ember_gemm_f32": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_linear_bf16": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _c_void, _c_size, _c_void, _c_void],
    "ember_linear_tc": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_linear_stream": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                            _c_void, _c_size, _c_void],
    "ember_linear_decode": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void,
                            _c_size, _c_void],
    "ember_clear_tails": [_c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_kv_store": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_void],
    "ember_attention_plain": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int,
                              _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void],
    "ember_attention_decode": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                               _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_void],
    "ember_attention_decode_ahead": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                                     _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                                     _c_int, _c_void, _c_void, _c_void],
    "ember_attention_decode_mma": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                                   _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                                   _c_int, _c_int, _c_void, _c_void, _c_void],
    "ember_attention_prefill": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int,
                                _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void],
    "ember_attention_prefill_tc": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int,
                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void],
    "ember_rmsnorm": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_float, _c_float, _c_int, _c_void],
    "ember_add_normed": [_c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_float, _c_float, _c_void],
    "ember_gated_act": [_c_void, _c_void, _c_int, _c_int, _c_int, _c_float, _c_float, _c_float, _c_int, _c_void],
    "ember_gated_group_norm": [_c_void, _c_void, ctypes.c_longlong, _c_void, _c_void, _c_int, _c_int, _c_int, _c_float,
                               _c_int, _c_int, _c_void],
    "ember_kv_store_v": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int,
                         _c_int, _c_int, _c_int, _c_void],
    "ember_attention_plain_v": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int,
                                _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_attention_prefill_kept": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                                     _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void],
    "ember_attention_decode_kept": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int,
                                    _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_void],
    "ember_conv_silu": [_c_void, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void,
                        _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_ssd_scan": [_c_void, _c_void, ctypes.c_longlong, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                       _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_int, _c_void],
    "ember_ssd_pieces": [_c_void, _c_void, ctypes.c_longlong, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                         _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void],
    "ember_moe_route": [_c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void],
    "ember_moe_gate_up": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _c_int, _c_int, _c_void],
    "ember_moe_down": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_void],
    "ember_pair_table_add": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int,
                             ctypes.c_longlong, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_void],
    "ember_rotate": [_c_void, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_void, ctypes.c_longlong, _c_int, _c_int, _c_int,
                     _c_int, _c_int, _c_int, _c_void, _c_void, _c_float, _c_int, _c_void],
    "ember_latent_rows": [_c_void, _c_int, _c_int, _c_void, _c_void, _c_int, _c_int, _c_float, _c_void, _c_float, _c_int,
                          _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void],
    "ember_head_linear": [_c_void, ctypes.c_longlong, _c_int, _c_int, _c_void, _c_void, ctypes.c_longlong, _c_int, _c_int,
                          _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_head_linear_bf16": [_c_void, ctypes.c_longlong, _c_int, _c_void, _c_void, ctypes.c_longlong, _c_int, _c_int, _c_int,
                               _c_int, _c_int, _c_void, _c_size, _c_void],
    "ember_latent_attention_plain": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int,
                                     _c_int, _c_int, _c_int, _c_float, _c_int, _c_void],
    "ember_latent_attention_mma": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int,
                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void],
    "ember_delta_rule": [_c_void, _c_void, ctypes.c_longlong, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void,
                         _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                         _c_int, _c_void],
    "ember_attention_plain_biased": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int,
                                     _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_void],
    "ember_attention_prefill_biased": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                                       _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void, _c_void,
                                       _c_void],
    "ember_attention_decode_biased": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int,
                                      _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void],
    "ember_add_branches": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_float, _c_void],
    "ember_qkv_norm": [_c_void, ctypes.c_longlong, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_float, _c_float, _c_int, _c_int, _c_int, _c_void],
    "ember_gate_mul": [_c_void, _c_void, ctypes.c_longlong, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_mlstm_gates": [_c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void],
    "ember_mlstm_scan": [_c_void, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                         _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void, _c_int, _c_void],
    "ember_mingru": [_c_void, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                     _c_void, _c_int, _c_int, _c_int, _c_int, _c_void, _c_int, _c_int, _c_void],
    "ember_sample": [_c_void, _c_void, _c_int, _c_int, _c_float, _c_int, _c_float, _c_u64, _c_void, _c_void, _c_u64, _c_void],
}


class KernelError(RuntimeError):
    pass


MOE_TILE_PAIRS = 48   # (token, choice) pairs from which the experts' products take tensor-core tiles (bfloat16)
SMALL_M = 16          # rows up to which the mma.sync weight-streaming product (linear_decode.cu) is used
STREAM_M = 64         # rows up to which the tcgen05 weight-streaming product (linear_stream.cu) is used above that
TC_MIN_M = 64         # rows above which the tcgen05 product is used (its tiles have 128 rows)


def _current_stream() -> int:
    """The handle of torch's current stream on the current device.  Asked for at every launch, so by the shortest
    way torch has (a launch costs the host a few microseconds in all, and a prompt's step is some 500 launches)."""
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is None:
        return torch.cuda.current_stream().cuda_stream
    return raw(torch.cuda.current_device())


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"element type {dtype} is neither float32 nor bfloat16")


def load_library() -> ctypes.CDLL:
    """Builds the library if needed and loads it; every failure is an error that says why."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is visible: this library runs models on a GPU only")
    major, minor = torch.cuda.get_device_capability()
    if major != 10:
        raise KernelError(f"the kernels are built for sm_100a; this device is sm_{major}{minor}")
    path = build.library_path()
    lib = ctypes.CDLL(path)
    lib.ember_last_error.restype = ctypes.c_char_p
    for name, args in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = _c_int
    lib.ember_umma_issue_probe.argtypes = [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void]
    lib.ember_umma_issue_probe.restype = _c_int
    lib.ember_wait_probe.argtypes = [_c_u64, _c_void]
    lib.ember_wait_probe.restype = _c_int
    lib.ember_set_option.argtypes = [_c_int, _c_int]
    lib.ember_set_option.restype = _c_int
    lib.ember_recurrence_piece.argtypes = []
    lib.ember_recurrence_piece.restype = _c_int
    lib.ember_recurrence_scratch.argtypes = [_c_int] * 6
    lib.ember_recurrence_scratch.restype = _c_size
    lib.ember_attention_decode_partials.argtypes = [_c_int] * 5
    lib.ember_attention_decode_partials.restype = _c_size
    lib.ember_ssd_scan_piece.argtypes = []
    lib.ember_ssd_scan_piece.restype = _c_int
    lib.ember_ssd_pieces_len.argtypes = []
    lib.ember_ssd_pieces_len.restype = _c_int
    lib.ember_ssd_scan_scratch.argtypes = [_c_int] * 5
    lib.ember_ssd_scan_scratch.restype = _c_size
    lib.ember_latent_attention_mma_scratch.argtypes = [_c_int] * 3
    lib.ember_latent_attention_mma_scratch.restype = _c_size
    lib.ember_delta_rule_scratch.argtypes = [_c_int] * 6
    lib.ember_delta_rule_scratch.restype = _c_size
    lib.ember_attention_decode_kept_scratch.argtypes = [_c_int] * 4
    lib.ember_attention_decode_kept_scratch.restype = _c_size
    lib.ember_mlstm_scan_scratch.argtypes = [_c_int] * 5
    lib.ember_mlstm_scan_scratch.restype = _c_size
    lib.ember_mingru_scratch.argtypes = [_c_int] * 3
    lib.ember_mingru_scratch.restype = _c_size
    for name in ("ember_tc_status", "ember_linear_decode_status", "ember_attention_decode_status",
                 "ember_attention_decode_mma_status"):
        getattr(lib, name).argtypes = []
        getattr(lib, name).restype = _c_int
    lib._path = path
    return lib


def decode_chunks(blocks: int, pairs: int, sms: int, slots: int, four_warps: bool) -> int:
    """Into how many chunks the decode attention cuts a context of `blocks` pages, each chunk a block of the
    launch, for `pairs` (token, head) pairs on a chip of `sms` SMs that holds `slots` two-warp blocks at once.

    The context is cut so that the launch fills the chip once: as many chunks as resident blocks per pair
    allow, at least two pages each (a block's fixed costs are then shared by 128 keys).  Pairs that fill the
    chip by themselves are not cut: their blocks write the output directly, with no partial results to
    merge.  (A block that waits for an SM starts its copies late: a step of 12 layers at batch 8 and a
    context of 900 to 1,024 0.557 against 0.593 ms.)

    four_warps (head size 64 on the tensor cores): while chunks of up to four pages (else of up to eight)
    are few enough for three blocks of four warps an SM to hold them all, the chunks are that long and a block
    has four warps, a page each at a time: fewer blocks to merge (none up to four pages), and four pages of a
    chunk on their way from the block's start.  (GPT-2 XL at batch 8: the first steps 1.312 -> 1.260 ms, the
    sweep to 1,024 tokens 1.433 -> 1.414.)"""
    n_chunks = max(1, min(slots // max(pairs, 1), -(-blocks // 2)))
    if four_warps and blocks > 2:
        for longest in (4, 8):
            n = -(-blocks // longest)
            if n <= 8 and n * pairs <= 3 * sms:
                return n
    return n_chunks


class CudaOps:
    name = "cuda-sm100a"

    def __init__(self, options=None):
        """`options`: a RuntimeOptions; None takes the defaults with the EMBER_* variables laid on top."""
        from ..options import RuntimeOptions
        self.options = options = options if options is not None else RuntimeOptions.from_env()
        self.lib = load_library()
        self._workspace = None
        self._partials = None          # scratch of the decode attention: partial results ...
        self._counters = None          # ... and its per-(token, head) counters, zero between calls
        self._retired = []             # outgrown scratch stays alive: captured graphs may still name it
        self.launches = 0
        self.sms = torch.cuda.get_device_properties(0).multi_processor_count
        self.decode_slots = 6 * self.sms   # blocks of the decode attention that are resident at once
        # What the switches are and why their defaults are what they are (all measured on GPT-2 XL's shapes):
        # cache_ahead: a decode attention asks the next layer's rows of the cache into L2.  Off: with the kernel
        #   that loads keys into registers the step's time did not change (0.5822 against 0.5820 ms of 12 layers);
        #   with the tensor-core kernel it grew (0.538 against 0.516 ms): a layer's rows and weights together do
        #   not stay in L2 that long, and the rows are then fetched twice.
        self.cache_ahead = options.cache_ahead
        # decode_mma: decode attention on the tensor cores where that kernel has an instantiation (head size 64
        #   or 128, up to 8 query heads to a key/value head); off takes the other kernel.
        self.decode_mma = options.decode_mma
        self._warm = None              # tensor announced by `warm` for the next product
        self._coming = []              # weight matrices announced by `announce_weights`, in the order their products run
        # warm: the second product of a feed-forward has its weights landed about a microsecond earlier with it
        #   (its blocks cannot be resident beside the first product's); a step of 12 layers 0.519 against 0.521 ms.
        self.warm_ahead = options.warm
        # gemm: products of more than STREAM_M rows go to cuBLASLt ("lt"), as ember.cpp's own go to cuBLAS, or
        #   ("tc"), above TC_MIN_M rows, to this library's tcgen05 kernel.  On GPT-2 XL's four products the
        #   library is ahead at 2,048 rows; at 16,384 rows the tcgen05 kernel reaches 95 % of it on the QKV product.
        self.gemm = options.gemm
        # lt_tune: the first product of a shape times the library's candidate algorithms; `deterministic` turns
        #   it off, so that the choice does not depend on a timing
        self.lt_tune = options.lt_tune
        self._lt_tuned = set()
        # linear_stream: products of SMALL_M + 1 to STREAM_M rows stream the weights through this library's tcgen05
        #   kernel with the operands swapped (linear_stream.cu); off sends them to cuBLASLt.
        self.linear_stream_on = options.linear_stream
        # attention: prefill attention with head size 64 on the tcgen05 kernel, or ("mma") on the mma.sync kernel
        #   (which takes every other head size anyway)
        self.attention_tc = options.attention == "tc"
        # attention_kept_fast: attention with kept first tokens or a value size of its own takes the mma.sync prompt
        #   kernel and the split one-token kernel where they have the sizes; False takes the plain kernel everywhere
        #   (a measurement switch: the twin that the two are compared with)
        self.attention_kept_fast = True
        # latent_fast: attention over cached low-rank rows in bfloat16 takes the tensor-core kernel where it has the
        #   sizes; False takes the plain kernel everywhere (the twin that it is compared with)
        self.latent_fast = True
        self.latent_pages_per_chunk = 0    # pages a block of its one-token form takes; 0: as many as fill the chip about twice
        # branch_streams: `side_by_side` runs independent branches of a one-token step on streams of their own
        self.branch_streams = options.branch_streams
        self._side_streams = []
        # op_timing, nvtx: per-launch CUDA events and NVTX ranges (see options.py); both off by default
        self.op_timing, self.nvtx = options.op_timing, options.nvtx
        self._timed = []
        # the three switches that the kernels' launch code reads (process-wide)
        for which, value in ((0, options.pdl), (1, options.decode_bulk), (2, options.decode_cluster)):
            self.lib.ember_set_option(which, 1 if value else 0)

    # ------------------------------------------------------------------ helpers
    def _call(self, name: str, *args, allow=()) -> int:
        timed = self.op_timing and not torch.cuda.is_current_stream_capturing()
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        if timed:
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
        rc = getattr(self.lib, name)(*args, _current_stream())
        if timed:
            end.record()
            self._timed.append((name, begin, end))
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
        if rc in allow:
            return rc
        self.launches += 1
        if rc != 0:
            raise KernelError(self.lib.ember_last_error().decode())
        return 0

    def op_times(self, reset: bool = True) -> dict:
        """With the `op_timing` option: {entry point: (launches, milliseconds)} since the last call, from CUDA
        events around every launch (an event between two launches keeps them from overlapping, so the sum is
        more than a step takes: read the shares).  Synchronizes with the device."""
        torch.cuda.synchronize()
        out: dict = {}
        for name, begin, end in self._timed:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + begin.elapsed_time(end))
        if reset:
            self._timed = []
        return out

    def _decode_scratch(self, n_partials: int, n_counters: int):
        if self._partials is None or self._partials.numel() < n_partials:
            self._retired.append(self._partials)
            self._partials = torch.empty(max(n_partials, 1 << 20), dtype=torch.float32, device="cuda")
        if self._counters is None or self._counters.numel() < n_counters:
            self._retired.append(self._counters)
            self._counters = torch.zeros(max(n_counters, 1 << 16), dtype=torch.int32, device="cuda")
        return self._partials, self._counters

    @staticmethod
    def _ptr(t):
        return None if t is None else t.data_ptr()

    @staticmethod
    def _dense(t: torch.Tensor, what: str) -> torch.Tensor:
        if not t.is_cuda or not t.is_contiguous():
            raise KernelError(f"{what} must be a contiguous CUDA tensor")
        return t

    def _lt_workspace(self) -> torch.Tensor:
        if self._workspace is None:
            self._workspace = torch.empty(_LT_WORKSPACE, dtype=torch.uint8, device="cuda")
        return self._workspace

    @staticmethod
    def _bias_bf16(bias: torch.Tensor) -> torch.Tensor:
        """The bfloat16 copy of a bias that cuBLASLt's epilogue reads.  It is kept on the bias tensor itself
        (made once, dies with it): a cache keyed by address would hand a freed model's copy to a new model
        whose bias landed on the same address."""
        copy = getattr(bias, "_ember_bf16", None)
        if copy is None or copy.shape != bias.shape or copy.device != bias.device:
            copy = bias.to(torch.bfloat16)
            bias._ember_bf16 = copy
        return copy

    # ------------------------------------------------------------------ rows
    def embed(self, tokens, positions, table, pos_table, token_src=None, ids=None, token_scale: float = 1.0):
        """Rows of the token table (plus rows of the position table) in float32.  With `token_src` and `ids`
        (int32, on the device) token t is ids[token_src[t]] where token_src[t] >= 0: an id that an earlier
        step's sampler left there.  `token_scale` multiplies the token's row alone, before the position's is added."""
        T, d = tokens.shape[0], table.shape[1]
        if pos_table is not None and (pos_table.dtype != table.dtype or pos_table.shape[1] != d):
            raise KernelError("embed: the position table must have the token table's type and width")
        if (token_src is None) != (ids is None):
            raise KernelError("embed: tokens from the device need both their rows and the ids")
        if ids is not None and (ids.dtype != torch.int32 or not ids.is_cuda or not ids.is_contiguous()):
            raise KernelError("embed: sampled ids are a contiguous int32 CUDA tensor")
        x = torch.empty((T, d), dtype=torch.float32, device=table.device)
        self._call("ember_embed", tokens.data_ptr(), positions.data_ptr(), self._dense(table, "token table").data_ptr(),
                   self._ptr(pos_table), x.data_ptr(), T, d, _code(table.dtype), self._ptr(token_src), self._ptr(ids),
                   0 if ids is None else ids.numel(), table.shape[0], float(token_scale))
        return x

    def warm(self, tensor) -> None:
        """Announces constants that a kernel soon after the next product reads (the weights of the product
        after it).  A hint: a small product's kernel asks them into L2 while it waits for its own input."""
        fits = tensor is not None and tensor.numel() * tensor.element_size() <= self.AHEAD_BYTES
        self._warm = tensor if self.warm_ahead and fits else None

    def announce_weights(self, weights) -> None:
        """Announces the weight matrices of the products to come, in the order they run (a block announces
        its own and the first of what follows it).  A hint: a product of 17 to 64 rows asks the matrix after
        its own into L2, so that the next product's ring refills from there and not from DRAM."""
        self._coming = [w for w in weights if w is not None]

    def _after(self, w):
        """The announced matrix that follows `w`, if it is worth asking into L2 (it fits there with room to spare)."""
        if not self.warm_ahead:
            return None
        for i, c in enumerate(self._coming[:-1]):
            if c.data_ptr() == w.data_ptr():
                nxt = self._coming[i + 1]
                return nxt if nxt.numel() * nxt.element_size() <= self.AHEAD_BYTES else None
        return None

    def layernorm(self, x, w, b, eps, out_dtype):
        """Layer norm of float32 rows."""
        rows, d = x.shape
        if x.dtype != torch.float32 or w.dtype != torch.float32 or b.dtype != torch.float32:
            raise KernelError("layernorm: input, gain and bias are float32")
        if w.shape[0] != d or b.shape[0] != d:
            raise KernelError(f"layernorm: width {d} with gain {tuple(w.shape)} and bias {tuple(b.shape)}")
        out = torch.empty((rows, d), dtype=out_dtype, device=x.device)
        self._call("ember_layernorm", self._dense(x, "layernorm input").data_ptr(), w.data_ptr(), b.data_ptr(),
                   out.data_ptr(), rows, d, float(eps), _code(out_dtype))
        return out

    AHEAD_BYTES = 48 << 20   # rows of one layer's cache that are worth asking into L2 a layer early

    TIMELINE_KERNELS = {1: "embed", 2: "layernorm", 3: "linear_decode", 4: "attention_decode", 5: "sample", 6: "linear_stream"}
    TIMELINE_FILES = ("elementwise", "linear_decode", "linear_stream", "attention_decode", "attention_decode_mma", "sampling")

    def timeline(self):
        """What the kernels of a library built with EMBER_TIMELINE=1 noted since the last call: a list of
        (nanoseconds, kernel name, mark, block, blocks of the launch, SM) sorted by time; mark 0 = the block
        started, 1 = its wait for the kernel in front returned, 2 = it ended (3: it ended after merging
        the partial results of a decode attention), 4 to 7 = places in between that the kernel's source
        names.  Synchronizes with the device."""
        import struct
        if not hasattr(self.lib, "ember_timeline_read_elementwise"):
            raise KernelError("this library was built without EMBER_TIMELINE=1")
        cap, out = 1 << 18, []
        buf = ctypes.create_string_buffer(cap * 24)
        for name in self.TIMELINE_FILES:
            fn = getattr(self.lib, f"ember_timeline_read_{name}")
            fn.argtypes, fn.restype = [_c_void, ctypes.c_uint], _c_int
            n = fn(ctypes.cast(buf, ctypes.c_void_p), cap)
            if n < 0:
                raise KernelError(f"timeline: reading the log of {name}.cu failed")
            for i in range(n):
                t, what, block, grid, sm = struct.unpack_from("<QIIII", buf, i * 24)
                if t:
                    out.append((t, self.TIMELINE_KERNELS.get(what >> 8, str(what >> 8)), what & 255, block, grid, sm))
        out.sort()
        return out

    def scale_cap(self, x, scale: float = 1.0, cap: float | None = None):
        """x <- scale * x, then (with a cap) cap * tanh(x / cap), in place on float32 values: a factor on
        the embedded rows, a cap on the logits."""
        if x.dtype != torch.float32:
            raise KernelError("scale_cap: float32 values (the residual stream, the logits)")
        self._call("ember_scale_cap_inplace", self._dense(x, "values").data_ptr(), x.numel(), float(scale),
                   0.0 if cap is None else float(cap))
        return x

    def take_tokens(self, tokens, token_src, ids, vocab_size: int) -> None:
        """tokens[i] = ids[token_src[i]] where token_src[i] >= 0: a step's tokens taken from an earlier
        step's sampled ids on the device."""
        if ids.dtype != torch.int32 or not ids.is_cuda or not ids.is_contiguous():
            raise KernelError("take_tokens: sampled ids are a contiguous int32 CUDA tensor")
        self._call("ember_take_tokens", tokens.data_ptr(), token_src.data_ptr(), ids.data_ptr(), tokens.shape[0],
                   ids.numel(), int(vocab_size))

    def gather_rows(self, x, rows, n_rows):
        out = torch.empty((n_rows, x.shape[1]), dtype=torch.float32, device=x.device)
        self._call("ember_gather_rows", self._dense(x, "rows").data_ptr(), rows.data_ptr(), out.data_ptr(), n_rows,
                   x.shape[1])
        return out

    # ------------------------------------------------------------------ products
    def linear(self, a, w, bias, act=None, residual=None, out_dtype=None):
        """y = a w^T (+ bias) (activation) (+ residual).  `w` is [out, in].  With a residual the
        sum is made in float32 into the residual's buffer, which is returned."""
        if act not in _ACT:
            raise KernelError(f"linear: activation {act!r}")
        warm, self._warm = self._warm, None
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise KernelError(f"linear: input width {K} does not match the weight's {tuple(w.shape)}")
        if a.dtype != w.dtype:
            raise KernelError(f"linear: input is {a.dtype}, weight is {w.dtype}")
        if bias is not None and (bias.dtype != torch.float32 or bias.shape[0] != N):
            raise KernelError("linear: the bias is float32 of the output's width")
        if residual is not None and (residual.dtype != torch.float32 or tuple(residual.shape) != (M, N)):
            raise KernelError("linear: the residual is float32 of the output's shape")
        self._dense(a, "linear input")
        self._dense(w, "linear weight")
        if w.dtype == torch.bfloat16 and K % 8:
            return self._linear_unaligned(a, w, bias, act, residual, out_dtype)
        if w.dtype == torch.float32:
            out = residual if residual is not None else torch.empty((M, N), dtype=torch.float32, device=a.device)
            self._call("ember_gemm_f32", a.data_ptr(), w.data_ptr(), self._ptr(bias), self._ptr(residual),
                       out.data_ptr(), M, N, K, _ACT[act])
            return out if out_dtype in (None, torch.float32) or residual is not None else out.to(out_dtype)
        target = torch.float32 if residual is not None else (out_dtype or torch.bfloat16)
        out = residual if residual is not None else torch.empty((M, N), dtype=target, device=a.device)
        # A matrix that fills L2 by itself (a vocabulary head) streams faster through the tcgen05 kernel from 9
        # rows on (GPT-2 XL's head at 16 rows: 34.7 against 48.0 microseconds; at 8 rows 32.9 against 27.4).
        big = w.numel() * 2 > (64 << 20) and M > 8 and self.linear_stream_on
        if act == "relu2" and M > TC_MIN_M and K % 8 == 0 and residual is None:
            # the library's product has no such epilogue: this library's tcgen05 product takes it (2,048 rows,
            # 2,048 -> 8,192: 60 microseconds against 35 and 40 more for the activation by itself)
            return self.linear_tc(a, w, bias, act, None, out)
        if act == "relu2" and not (M <= SMALL_M and K % 8 == 0 and K <= 16384 and not big):
            # of the other products only the small one has this activation in its epilogue: the rest run plain, the
            # activation after them
            if residual is not None:
                raise KernelError("linear: an activation after the product cannot follow a residual sum")
            out = self.linear(a, w, bias, None, None, out_dtype)
            self._call("ember_act_inplace", out.data_ptr(), out.numel(), _ACT[act], _code(out.dtype))
            return out
        if M <= SMALL_M and K % 8 == 0 and K <= 16384 and not big:
            # (Only a matrix that a part announced with `warm` is asked into L2 here.  Every product asking for the
            # next announced matrix paid at 8 rows once, 1.556 -> 1.512 ms a step of GPT-2 XL, and costs since the
            # launches spread over the chip: 1.307 against 1.280 ms.)
            self._call("ember_linear_decode", a.data_ptr(), w.data_ptr(), self._ptr(bias), self._ptr(residual), out.data_ptr(),
                       M, N, K, _ACT[act], _code(target), None if warm is None else warm.data_ptr(),
                       0 if warm is None else warm.numel() * warm.element_size() // 16 * 16)
            return out
        if self.linear_stream_on and M <= STREAM_M and K % 8 == 0:
            return self.linear_stream(a, w, bias, act, residual, out, warm=warm if warm is not None else self._after(w))
        # an output width that is no multiple of 8 (a vocabulary of 50,257) leaves the library only unaligned,
        # slow kernels (167 against 50 microseconds for the head at 64 rows): those products take the tcgen05 kernel
        if K % 8 == 0 and ((self.gemm == "tc" and M > TC_MIN_M) or N % 8 != 0):
            return self.linear_tc(a, w, bias, act, residual, out)
        fused = _ACT[act] if act != "gelu_erf" else 0
        ws = self._lt_workspace()
        # the first product of a shape times the library's candidates into a scratch output (outside any capture)
        shape = (M, N, K, fused, bias is not None, residual is not None, target)
        scratch = None
        # (large products only, and a bounded number of shapes: timing costs a few milliseconds a shape)
        if (self.lt_tune and M >= 64 and shape not in self._lt_tuned and len(self._lt_tuned) < 512
                and not torch.cuda.is_current_stream_capturing()):
            self._lt_tuned.add(shape)
            scratch = torch.empty_like(out)
        self._call("ember_linear_bf16", a.data_ptr(), w.data_ptr(), self._ptr(bias),
                   None if bias is None else self._bias_bf16(bias).data_ptr(), self._ptr(residual), out.data_ptr(),
                   M, N, K, fused, _code(target), ws.data_ptr(), ws.numel(), self._ptr(scratch))
        if act == "gelu_erf":
            self._call("ember_act_inplace", out.data_ptr(), out.numel(), _ACT[act], _code(target))
        return out

    def _linear_unaligned(self, a, w, bias, act, residual, out_dtype):
        """A bfloat16 product whose rows are no multiples of 16 bytes (K % 8 != 0), which none of the bfloat16 kernels
        reads: the float32 product on the same values (bfloat16 widens exactly, the sums are float32 as theirs are),
        its result rounded as theirs would be.  Slow; a model of such sizes still runs in both compute types."""
        wide = getattr(w, "_ember_f32", None)          # kept on the weight itself: made once, dies with it
        if wide is None or wide.shape != w.shape or wide.device != w.device:
            wide = w.float()
            w._ember_f32 = wide
        rows = a.float()
        M, K = a.shape
        N = w.shape[0]
        out = residual if residual is not None else torch.empty((M, N), dtype=torch.float32, device=a.device)
        self._call("ember_gemm_f32", rows.data_ptr(), wide.data_ptr(), self._ptr(bias), self._ptr(residual), out.data_ptr(),
                   M, N, K, _ACT[act])
        if residual is not None:
            return out
        return out.to(out_dtype or torch.bfloat16)

    def linear_tc(self, a, w, bias, act, residual, out, tile_n: int = 0):
        """The tcgen05 product with its epilogue (bias, activation, float32 residual sum) into `out`."""
        M, K = a.shape
        self._call("ember_linear_tc", a.data_ptr(), w.data_ptr(), self._ptr(bias), self._ptr(residual), out.data_ptr(),
                   M, w.shape[0], K, _ACT[act], _code(out.dtype), tile_n)
        return out

    def linear_stream(self, a, w, bias, act, residual, out, k_split: int = 0, stages: int = 0, warm=None):
        """The tcgen05 weight-streaming product for up to 64 rows with its epilogue into `out`; `k_split` and
        `stages` 0 let the kernel choose how many blocks share a tile and how deep its ring is; `warm`: a tensor
        that the launch asks into L2 (the next product's weights)."""
        M, K = a.shape
        self._call("ember_linear_stream", a.data_ptr(), w.data_ptr(), self._ptr(bias), self._ptr(residual), out.data_ptr(),
                   M, w.shape[0], K, _ACT[act], _code(out.dtype), int(k_split), int(stages),
                   None if warm is None else warm.data_ptr(), 0 if warm is None else warm.numel() * warm.element_size() // 16 * 16)
        return out

    def umma_issue_probe(self, m: int, n: int, iters: int = 512, elected: bool = True, commit_every: int = 0, wait_too: bool = False):
        """(cycles to issue, cycles until complete) per `tcgen05.mma` of M = m, N = n, K = 16, issued from a single
        thread's branch or by a converged warp with elect.sync (umma_probe.cu).  A measurement for the notes."""
        out = torch.zeros(3, dtype=torch.int64, device="cuda")
        self._call("ember_umma_issue_probe", int(m), int(n), int(iters), 1 if elected else 0, int(commit_every), 1 if wait_too else 0, out.data_ptr())
        issue, done, ended = out.tolist()
        if not ended:
            raise KernelError("umma_issue_probe: the products did not complete within the wait's limit")
        return issue / iters, done / iters

    def wait_probe(self, limit_ns: int = 1_000_000) -> None:
        """Launches the kernel whose only wait nothing ends (wait_probe.cu): it gives up after `limit_ns`
        and leaves code 31 in the status word, which the next `check()` raises for.  For tests of the
        kernels' bounded waits; nothing faults or hangs."""
        self._call("ember_wait_probe", int(limit_ns))

    def check(self) -> None:
        """Raises if a kernel with bounded waits gave up since the last call.  The caller has
        synchronized with the device (it has just read a step's results)."""
        if self.lib.ember_linear_decode_status():
            raise KernelError("linear_decode: a block gave up waiting for its weight copies; the results of that launch are not valid")
        if self.lib.ember_attention_decode_status() or self.lib.ember_attention_decode_mma_status():
            raise KernelError("attention_decode: a block gave up waiting for its copies of keys and values; the results of that launch are not valid")
        code = self.lib.ember_tc_status()
        if code:
            kernel = "linear_tc" if code < 10 else ("attention_prefill_tc" if code < 20 else
                                                    ("linear_stream" if code < 30 else "wait_probe"))
            role = {31: "the probe's wait, as it is meant to",1: "the TMA producer", 2: "the product issuer", 3: "the epilogue", 4: "copies in flight",
                    11: "the TMA loader", 12: "the product issuer", 13: "the softmax warps",
                    21: "the TMA producer", 22: "the product issuer", 23: "the epilogue", 24: "copies in flight"}.get(code, code)
            raise KernelError(f"{kernel}: a wait ran out ({role}); the results of that launch are not valid")

    # ------------------------------------------------------------------ cache and attention
    def clear_tails(self, group, tails) -> None:
        """Zeroes, in every key and value tensor of a cache group, the rows from `row` on of each page
        named in tails [n, 2] = (page, row) (page < 0: nothing)."""
        need = group.need
        tables = getattr(group, "_tensor_tables", None)
        if tables is None:      # the addresses of the group's tensors, once (keys and values apart where their rows differ)
            sets = [(list(group.k) + list(group.v), need.head_dim)] if need.v_dim == need.head_dim else \
                [(list(group.k), need.head_dim), (list(group.v), need.v_dim)]
            tables = group._tensor_tables = [
                (torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=tensors[0].device), row)
                for tensors, row in sets]
        for table, row in tables:
            self._call("ember_clear_tails", table.data_ptr(), table.numel(), tails.data_ptr(), tails.shape[0], need.kv_heads,
                       row, group.k[0].element_size())

    def kv_store(self, qkv, cache, plan, n_heads, kv_heads, head_dim):
        if qkv.dtype != cache.k.dtype:
            raise KernelError(f"kv_store: activations are {qkv.dtype}, the cache is {cache.k.dtype}")
        self._call("ember_kv_store", self._dense(qkv, "qkv").data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                   plan.positions.data_ptr(), plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(),
                   plan.pages[cache.group_index].data_ptr(), plan.max_blocks, plan.T, n_heads, kv_heads, head_dim,
                   _code(qkv.dtype))

    def attention(self, qkv, cache, plan, n_heads, kv_heads, head_dim, scale, window, out_dtype, store=False,
                  keep_first=None, value_dim=None, slopes=None, sinks=None, chunk=0, head_scales=None,
                  head_scales_positive=True):
        """Causal attention of the step's tokens over the cache.  With `store` their own keys and
        values are written into the cache first (in the same launch where a kernel can).
        float32: the plain kernel, whose sums depend on positions alone.  bfloat16: one token per
        sequence takes the split decode kernel; anything else the tensor-core prefill kernel, or
        the plain kernel for head sizes that one has no instantiation for.
        keep_first / value_dim (a mixer that keeps a sequence's first positions visible beside its
        window, or whose values have a row size of their own): the plain kernel, which knows both and
        every head size, or for prompts in bfloat16 the mma.sync kernel where it has the head size.
        slopes (float32 per query head): the score of a key loses slopes[h] times its distance to the query.
        sinks (float32 per query head): the softmax's denominator also holds exp(sinks[h]), a term without a
        key or a value.  Both go the way of keep_first / value_dim.
        chunk > 0 (in place of a window): a query at position p sees key j <= p only if floor(j / chunk) =
        floor(p / chunk).  head_scales (float32 per query head): one more factor on a head's scores; the
        tensor-core prompt kernel takes it where every factor is above zero (`head_scales_positive`).  Both go
        the same way too."""
        if qkv.dtype != cache.k.dtype or out_dtype != qkv.dtype:
            raise KernelError("attention: activations, cache and output have one element type")
        self._dense(qkv, "qkv")
        for name, t in (("slopes", slopes), ("sinks", sinks), ("head_scales", head_scales)):
            if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != (n_heads,) or not t.is_cuda):
                raise KernelError(f"attention: {name} are float32 values, one a query head")
        if chunk < 0 or (chunk and (window or keep_first)):
            raise KernelError(f"attention: chunk {chunk} beside window {window} and {keep_first} kept positions")
        if keep_first is not None or value_dim is not None or slopes is not None or sinks is not None or chunk or head_scales is not None:
            return self._attention_kept(qkv, cache, plan, n_heads, kv_heads, head_dim, scale, window, out_dtype, store,
                                        int(keep_first or 0), head_dim if value_dim is None else int(value_dim), slopes, sinks,
                                        int(chunk), head_scales, head_scales_positive)
        out = torch.empty((plan.T, n_heads * head_dim), dtype=out_dtype, device=qkv.device)
        pages = plan.pages[cache.group_index]
        if qkv.dtype == torch.bfloat16 and plan.all_single:
            if plan.T != plan.n:      # the decode kernels take token t for sequence t of the step
                raise KernelError("attention: a step of one token each has as many tokens as sequences")
            blocks = min(plan.max_blocks, max(1, -(-plan.max_end // 64)))
            mma = self.decode_mma and head_dim in (64, 128) and n_heads // kv_heads <= 8
            pairs = plan.T * (kv_heads if mma else n_heads)   # the tensor-core kernel takes a group of heads a block
            n_chunks = decode_chunks(blocks, pairs, self.sms, self.decode_slots, mma and head_dim == 64)
            per_chunk = -(-blocks // n_chunks)
            n_partials = self.lib.ember_attention_decode_partials(plan.T, n_heads, head_dim, blocks, per_chunk)
            partials, counters = self._decode_scratch(n_partials, plan.T * n_heads)
            # The layer that attends next from the same group of the cache reads the same rows of its own
            # pages: while they all fit in L2 beside a layer's weights, this launch asks them there.
            ahead = getattr(cache, "following", None) if self.cache_ahead else None
            rows_bytes = plan.T * blocks * 64 * kv_heads * head_dim * 2 * 2
            ahead_k, ahead_v = (ahead[0].data_ptr(), ahead[1].data_ptr()) if ahead and rows_bytes <= self.AHEAD_BYTES else (0, 0)
            if self.decode_mma:
                rc = self._call("ember_attention_decode_mma", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                out.data_ptr(), partials.data_ptr(), counters.data_ptr(), plan.positions.data_ptr(),
                                plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(), pages.data_ptr(), plan.max_blocks,
                                blocks, cache.k.shape[0], plan.T, n_heads, kv_heads, head_dim, float(scale), int(window),
                                per_chunk, 1 if store else 0, ahead_k, ahead_v, allow=(2,))
                if rc == 0:
                    return out
            self._call("ember_attention_decode_ahead", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                       out.data_ptr(), partials.data_ptr(), counters.data_ptr(), plan.positions.data_ptr(),
                       plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(), pages.data_ptr(), plan.max_blocks, blocks,
                       plan.T, n_heads, kv_heads, head_dim, float(scale), int(window), per_chunk, 1 if store else 0,
                       ahead_k, ahead_v)
            return out
        if store:
            self.kv_store(qkv, cache, plan, n_heads, kv_heads, head_dim)
        if qkv.dtype == torch.bfloat16 and scale > 0 and self.attention_tc:
            rc = self._call("ember_attention_prefill_tc", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                            out.data_ptr(), plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(), plan.seq_new.data_ptr(),
                            plan.cu_new.data_ptr(), pages.data_ptr(), plan.max_blocks, plan.n, plan.max_new, plan.T,
                            cache.k.shape[0], n_heads, kv_heads, head_dim, float(scale), int(window), allow=(2,))
            if rc == 0:
                return out
        if qkv.dtype == torch.bfloat16 and scale > 0:
            rc = self._call("ember_attention_prefill", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                            out.data_ptr(), plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(), plan.seq_new.data_ptr(),
                            plan.cu_new.data_ptr(), pages.data_ptr(), plan.max_blocks, plan.n, plan.max_new, n_heads,
                            kv_heads, head_dim, float(scale), int(window), allow=(2,))
            if rc == 0:
                return out
        self._call("ember_attention_plain", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                   out.data_ptr(), plan.positions.data_ptr(), plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(),
                   pages.data_ptr(), plan.max_blocks, plan.T, n_heads, kv_heads, head_dim,
                   float(scale), int(window), _code(qkv.dtype))
        return out

    def _attention_kept(self, qkv, cache, plan, n_heads, kv_heads, hd, scale, window, out_dtype, store, keep_first, vd,
                        slopes=None, sinks=None, chunk=0, head_scales=None, head_scales_positive=True):
        if qkv.shape[1] != (n_heads + kv_heads) * hd + kv_heads * vd:
            raise KernelError(f"attention: rows of {qkv.shape[1]} values are not q | k | v of {n_heads} x {hd}, "
                              f"{kv_heads} x {hd} and {kv_heads} x {vd}")
        if tuple(cache.v.shape[1:]) != (kv_heads, 64, vd) or tuple(cache.k.shape[1:]) != (kv_heads, 64, hd):
            raise KernelError("attention: the cache's pages do not have the mixer's head sizes")
        out = torch.empty((plan.T, n_heads * vd), dtype=out_dtype, device=qkv.device)
        pages = plan.pages[cache.group_index]
        if store:
            self._call("ember_kv_store_v", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(), plan.positions.data_ptr(),
                       plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(), pages.data_ptr(), plan.max_blocks, plan.T,
                       n_heads, kv_heads, hd, vd, _code(qkv.dtype))
        fast = self.attention_kept_fast and qkv.dtype == torch.bfloat16
        if fast and plan.all_single and plan.T == plan.n:
            # one token each: the visible keys in chunks of 128, a block a chunk and key/value head, then the merge
            max_keys = min(keep_first + window, plan.max_end) if window > 0 else (min(chunk, plan.max_end) if chunk else plan.max_end)
            scratch = torch.empty(self.lib.ember_attention_decode_kept_scratch(plan.T, n_heads, vd, max_keys),
                                  dtype=torch.float32, device=qkv.device)
            rc = self._call("ember_attention_decode_chunked", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                            out.data_ptr(), scratch.data_ptr(), plan.positions.data_ptr(), plan.seq_slot.data_ptr(),
                            pages.data_ptr(), plan.max_blocks, plan.T, n_heads, kv_heads, hd, vd, float(scale), int(window),
                            keep_first, int(max_keys), self._ptr(slopes), self._ptr(sinks), chunk, self._ptr(head_scales),
                            allow=(2,))
            if rc == 0:
                self.launches += 1      # (the merge)
                return out
        if fast and vd == hd and hd % 16 == 0 and hd <= 128 and scale > 0 and not plan.all_single and head_scales_positive:
            rc = self._call("ember_attention_prefill_chunked", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                            out.data_ptr(), plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(), plan.seq_new.data_ptr(),
                            plan.cu_new.data_ptr(), pages.data_ptr(), plan.max_blocks, plan.n, plan.max_new, n_heads,
                            kv_heads, hd, float(scale), int(window), keep_first, self._ptr(slopes), self._ptr(sinks), chunk,
                            self._ptr(head_scales), allow=(2,))
            if rc == 0:
                return out
        self._call("ember_attention_plain_chunked", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(), out.data_ptr(),
                   plan.positions.data_ptr(), plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(), pages.data_ptr(),
                   plan.max_blocks, plan.T, n_heads, kv_heads, hd, float(scale), int(window), vd, keep_first,
                   self._ptr(slopes), self._ptr(sinks), chunk, self._ptr(head_scales), _code(qkv.dtype))
        return out

    # ------------------------------------------------------------------ branches side by side
    def side_by_side(self, branches):
        """Runs independent pieces of a step (callables that launch kernels and return their results) and returns
        their results in order.  With `branch_streams` the first runs on the current stream and every other one on a
        stream of its own that waits for what the current stream has queued so far; the current stream then waits
        for all of them.  Inside a captured graph the branches become parallel paths of the graph.  A branch must
        read only what was queued before the call and write only what the others do not touch."""
        if not self.branch_streams or len(branches) < 2:
            return [run() for run in branches]
        while len(self._side_streams) < len(branches) - 1:
            self._side_streams.append(torch.cuda.Stream())
        main = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(main)
        results, joins = [None] * len(branches), []
        for k, run in enumerate(branches[1:], 1):
            side = self._side_streams[k - 1]
            side.wait_event(fork)
            with torch.cuda.stream(side):
                results[k] = run()
                done = torch.cuda.Event()
                done.record(side)
            joins.append(done)
        results[0] = branches[0]()
        for done in joins:
            main.wait_event(done)
        return results

    # ------------------------------------------------------------------ RMS norm, gates
    def rmsnorm(self, x, w, eps, out_dtype, offset=0.0):
        """x / sqrt(mean(x^2) + eps) * (offset + w) of float32 rows."""
        rows, d = x.shape
        if x.dtype != torch.float32 or w.dtype != torch.float32 or w.shape[0] != d:
            raise KernelError("rmsnorm: float32 rows and a float32 gain of their width")
        out = torch.empty((rows, d), dtype=out_dtype, device=x.device)
        self._call("ember_rmsnorm", self._dense(x, "rmsnorm input").data_ptr(), w.data_ptr(), out.data_ptr(), rows, d,
                   float(eps), float(offset), _code(out_dtype))
        return out

    def add_normed(self, x, branches, w, eps, offset=0.0):
        """x += rmsnorm(sum of factor * rows over `branches`) in place, one launch.  Every branch is float32
        [rows, width]; its rows may lie apart (a slice of a wider tensor), their values may not."""
        rows, d = x.shape
        if x.dtype != torch.float32 or not x.is_contiguous() or w.dtype != torch.float32 or w.shape[0] != d:
            raise KernelError("add_normed: a contiguous float32 stream and a float32 gain of its width")
        n = len(branches)
        if not 1 <= n <= 16:
            raise KernelError(f"add_normed: {n} branches (1 to 16)")
        for t, _ in branches:
            if t.dtype != torch.float32 or tuple(t.shape) != (rows, d) or t.stride(1) != 1 or not t.is_cuda:
                raise KernelError("add_normed: every branch is float32 [rows, width] with contiguous rows")
        ptrs = (_c_void * n)(*[t.data_ptr() for t, _ in branches])
        strides = (ctypes.c_longlong * n)(*[t.stride(0) for t, _ in branches])
        factors = (_c_float * n)(*[float(f) for _, f in branches])
        self._call("ember_add_normed", x.data_ptr(), ctypes.cast(ptrs, _c_void), ctypes.cast(strides, _c_void),
                   ctypes.cast(factors, _c_void), n, w.data_ptr(), rows, d, float(eps), float(offset))
        return x

    _GATES = {"silu": 0, "clamped_sigmoid": 1}

    def gated_act(self, gu, activation, limit=0.0, alpha=1.0, shift=0.0):
        """Rows of [gate | up] -> act(gate) * up, see parts/mlp.py for the two forms."""
        if activation not in self._GATES:
            raise KernelError(f"gated_act: activation {activation!r}")
        rows, n2 = gu.shape
        if n2 % 2:
            raise KernelError("gated_act: rows of gate | up have an even length")
        out = torch.empty((rows, n2 // 2), dtype=gu.dtype, device=gu.device)
        self._call("ember_gated_act", self._dense(gu, "gate | up").data_ptr(), out.data_ptr(), rows, n2 // 2,
                   self._GATES[activation], float(limit), float(alpha), float(shift), _code(gu.dtype))
        return out

    # ------------------------------------------------------------------ Mamba-2
    def conv_silu(self, proj, col0, channels, conv_w, conv_b, conv_state, plan, act="silu"):
        """silu (act "none": nothing) of the causal convolution (conv_w [channels, taps], the last tap on the current token) of
        `channels` columns from col0 of `proj`, per sequence of the step; conv_state [slots, taps - 1, channels]
        float32 carries the rows before the step and is advanced."""
        taps = conv_w.shape[1]
        if conv_w.shape[0] != channels or conv_b.shape[0] != channels or col0 + channels > proj.shape[1]:
            raise KernelError("conv_silu: the filter, its bias and the columns do not fit")
        if taps > 1 and (conv_state is None or tuple(conv_state.shape[1:]) != (taps - 1, channels) or conv_state.dtype != torch.float32):
            raise KernelError("conv_silu: the state is float32 [slots, taps - 1, channels]")
        self._dense(proj, "conv input")
        out = torch.empty((plan.T, channels), dtype=proj.dtype, device=proj.device)
        if act not in ("silu", "none"):
            raise KernelError(f"conv_silu: activation {act!r}")
        self._call("ember_conv_act", proj.data_ptr(), proj.stride(0), int(col0), int(channels), int(taps), conv_w.data_ptr(),
                   conv_b.data_ptr(), self._ptr(conv_state), out.data_ptr(), plan.token_seq.data_ptr(),
                   plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(), plan.cu_new.data_ptr(), plan.T, plan.n,
                   max(int(plan.max_new), 1), 1 if plan.all_single else 0, _code(proj.dtype), 0 if act == "silu" else 1)
        return out

    SSD_PIECES_FROM = 128   # new tokens of a step's longest sequence from which the recurrence runs as matrix products

    def ssd_scan(self, xbc, proj, dt_col, dt_bias, a_log, skip, state, plan, heads, vdim, groups, n_state,
                 tensor_cores=None):
        """The recurrence of parts/ssm.py over the step's sequences: xbc [T, x | B | C], the raw step sizes in
        `heads` columns from dt_col of `proj`, state float32 [slots, heads, vdim, n_state] (advanced); float32 y."""
        inner = heads * vdim
        if xbc.shape[1] != inner + 2 * groups * n_state or xbc.dtype != proj.dtype:
            raise KernelError("ssd_scan: rows of x | B | C in the projection's element type")
        if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, vdim, n_state):
            raise KernelError("ssd_scan: the state is float32 [slots, heads, vdim, states]")
        self._dense(xbc, "x | B | C")
        y = torch.empty((plan.T, inner), dtype=torch.float32, device=xbc.device)
        # prompts in bfloat16: pieces of 64 tokens as matrix products on the tensor cores, where the sizes have
        # an instantiation (tensor_cores: None lets the step's shape decide, False takes the scalar scan)
        if tensor_cores is None:
            tensor_cores = plan.max_new >= self.SSD_PIECES_FROM
        if tensor_cores and xbc.dtype == torch.bfloat16:
            pieces = max(1, -(-plan.max_new // self.lib.ember_ssd_pieces_len()))
            scratch = torch.empty(self.lib.ember_ssd_scan_scratch(plan.n, max(pieces, 2), heads, vdim, n_state),
                                  dtype=torch.float32, device=xbc.device)
            rc = self._call("ember_ssd_pieces", xbc.data_ptr(), proj.data_ptr(), proj.stride(0), int(dt_col),
                            dt_bias.data_ptr(), a_log.data_ptr(), skip.data_ptr(), state.data_ptr(), y.data_ptr(),
                            plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(), plan.cu_new.data_ptr(), plan.n, heads, vdim,
                            groups, n_state, pieces, scratch.data_ptr(), allow=(2,))
            if rc == 0:
                self.launches += 2
                return y
        # a step with a long sequence scans every sequence in pieces side by side (see ssm.cu)
        piece = self.lib.ember_ssd_scan_piece()
        pieces = -(-plan.max_new // piece) if plan.max_new >= 2 * piece else 1
        scratch = None
        if pieces > 1:
            scratch = torch.empty(self.lib.ember_ssd_scan_scratch(plan.n, pieces, heads, vdim, n_state), dtype=torch.float32,
                                  device=xbc.device)
        self._call("ember_ssd_scan", xbc.data_ptr(), proj.data_ptr(), proj.stride(0), int(dt_col), dt_bias.data_ptr(),
                   a_log.data_ptr(), skip.data_ptr(), state.data_ptr(), y.data_ptr(), plan.seq_slot.data_ptr(),
                   plan.seq_start.data_ptr(), plan.cu_new.data_ptr(), plan.n, heads, vdim, groups, n_state, pieces,
                   self._ptr(scratch), _code(xbc.dtype))
        return y

    def gated_group_norm(self, y, proj, z_col, w, parts, eps, out_dtype, gate_first=True, gate="silu"):
        """unit(y * silu(z)) * w with the root mean square over each of `parts` equal pieces of a row; z: the
        columns from z_col of `proj`.  gate_first False: unit(y) * w * silu(z), the gate after the norm.
        gate "sigmoid": sigmoid(z) in place of silu(z)."""
        if gate not in ("silu", "sigmoid"):
            raise KernelError(f"gated_group_norm: gate {gate!r}")
        rows, n = y.shape
        if y.dtype != torch.float32 or proj.dtype != out_dtype or z_col + n > proj.shape[1] or w.shape[0] != n:
            raise KernelError("gated_group_norm: float32 y, the gate in the output's element type, a gain of y's width")
        out = torch.empty((rows, n), dtype=out_dtype, device=y.device)
        z = proj[:, z_col:]
        self._call("ember_gated_group_norm", self._dense(y, "y").data_ptr(), z.data_ptr(), proj.stride(0), w.data_ptr(),
                   out.data_ptr(), rows, n, int(parts), float(eps), (1 if gate_first else 0) | (2 if gate == "sigmoid" else 0),
                   _code(out_dtype))
        return out


    # ------------------------------------------------------------------ branches with norms of their own, gates
    def add_branches(self, x, branches, gain, eps):
        """x += gain * sum of factor * b over `branches` in place, one launch.  A branch is (rows, factor) or
        (rows, factor, w): with w (a float32 gain of the row's width) the rows are divided by their root mean square
        and multiplied by w first.  gain: float32 per channel, or None."""
        rows, d = x.shape
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise KernelError("add_branches: a contiguous float32 stream")
        n = len(branches)
        if not 1 <= n <= 8:
            raise KernelError(f"add_branches: {n} branches (1 to 8)")
        norms = []
        for b in branches:
            t, w = b[0], (b[2] if len(b) > 2 else None)
            if t.dtype != torch.float32 or tuple(t.shape) != (rows, d) or t.stride(1) != 1 or not t.is_cuda:
                raise KernelError("add_branches: every branch is float32 [rows, width] with contiguous rows")
            if w is not None and (w.dtype != torch.float32 or tuple(w.shape) != (d,)):
                raise KernelError("add_branches: a branch's gain is float32 of the row's width")
            norms.append(w)
        if gain is not None and (gain.dtype != torch.float32 or tuple(gain.shape) != (d,)):
            raise KernelError("add_branches: the gain is float32 of the row's width")
        ptrs = (_c_void * n)(*[b[0].data_ptr() for b in branches])
        strides = (ctypes.c_longlong * n)(*[b[0].stride(0) for b in branches])
        factors = (_c_float * n)(*[float(b[1]) for b in branches])
        gains = (_c_void * n)(*[self._ptr(w) for w in norms])
        self._call("ember_add_branches", x.data_ptr(), ctypes.cast(ptrs, _c_void), ctypes.cast(strides, _c_void),
                   ctypes.cast(factors, _c_void), ctypes.cast(gains, _c_void), n, self._ptr(gain), rows, d, float(eps))
        return x

    def qkv_norm(self, proj, positions, heads, kv_heads, head_dim, value_dim, out_dtype, q_gain=None, k_gain=None,
                 unit_values=False, eps=0.0, temp_coef=0.0, temp_every=1):
        """The first columns of `proj` (q | k | v) as packed rows of `out_dtype`: q and k each divided by their root mean
        square over the whole row of heads and multiplied by a gain (where one is given), q then by the temperature
        1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) of its position p, and every value head divided by its own root
        mean square (`unit_values`)."""
        T = proj.shape[0]
        q_w, k_w = heads * head_dim, kv_heads * head_dim
        width = q_w + k_w + kv_heads * value_dim
        if proj.shape[1] < width or proj.stride(1) != 1:
            raise KernelError("qkv_norm: rows too short for q | k | v")
        for name, g, n in (("q", q_gain, q_w), ("k", k_gain, k_w)):
            if g is not None and (g.dtype != torch.float32 or tuple(g.shape) != (n,)):
                raise KernelError(f"qkv_norm: the gain of {name} is float32 of its width")
        out = torch.empty((T, width), dtype=out_dtype, device=proj.device)
        self._call("ember_qkv_norm", proj.data_ptr(), proj.stride(0), out.data_ptr(), positions.data_ptr(), self._ptr(q_gain),
                   self._ptr(k_gain), T, q_w, k_w, kv_heads, value_dim, 1 if unit_values else 0, float(eps), float(temp_coef),
                   int(temp_every), _code(proj.dtype), _code(out_dtype))
        return out

    def gate_mul(self, a, proj, z_col, gate="sigmoid"):
        """a * gate(z), z the columns from z_col of `proj`; gate "sigmoid" or "silu"."""
        rows, n = a.shape
        if gate not in ("silu", "sigmoid") or z_col + n > proj.shape[1] or proj.shape[0] != rows:
            raise KernelError("gate_mul: the gate's columns do not fit")
        out = torch.empty_like(a)
        z = proj[:, z_col:]
        self._call("ember_gate_mul", self._dense(a, "gated rows").data_ptr(), z.data_ptr(), proj.stride(0), out.data_ptr(), rows, n,
                   1 if gate == "sigmoid" else 0, _code(a.dtype), _code(proj.dtype))
        return out

    # ------------------------------------------------------------------ mLSTM, minGRU
    def mlstm_gates(self, h, w, bias, heads, cap):
        """float32 [T, 2 * heads]: the heads' log input gates cap * tanh((h w_i + b_i) / cap), then their log forget gates
        logsigmoid(cap * tanh((h w_f + b_f) / cap)); w [2 * heads, width] in h's element type, bias float32."""
        T, width = h.shape
        if w.dtype != h.dtype or tuple(w.shape) != (2 * heads, width) or bias.dtype != torch.float32 or bias.shape[0] != 2 * heads:
            raise KernelError("mlstm_gates: the gates' rows in the input's element type and a float32 bias")
        gates = torch.empty((T, 2 * heads), dtype=torch.float32, device=h.device)
        self._call("ember_mlstm_gates", self._dense(h, "mixer input").data_ptr(), self._dense(w, "gate rows").data_ptr(),
                   bias.data_ptr(), gates.data_ptr(), T, heads, width, float(cap), _code(h.dtype))
        return gates

    def _pieces(self, longest: int, blocks_per_piece: int, resident: int | None = None) -> int:
        """Into how many pieces a step's longest sequence is cut when a recurrence walks pieces side by side (twice:
        once from nothing, once from each piece's start state): none below 256 tokens.  Without `resident`: pieces of
        128, 64 or 32 tokens, the longest that still give the launch four blocks for every SM.  With `resident` (the
        blocks of the kernel that the chip holds at once): the count that makes waves of blocks x a piece's tokens x
        two walks smallest, a piece counted 16 tokens longer than it is for what its start and end cost; a launch
        that ends a little into a second wave takes twice as long as one that just fits the first."""
        if longest < 256:
            return 1
        if resident is None:
            for piece in (128, 64, 32):
                pieces = -(-longest // piece)
                if pieces * blocks_per_piece >= 4 * self.sms or piece == 32:
                    return pieces
        best, best_cost = 1, -(-blocks_per_piece // resident) * (longest + 16)
        for pieces in range(3, longest // 32 + 1):
            cost = -(-pieces * blocks_per_piece // resident) * (-(-longest // pieces) + 16) * 2
            if cost < best_cost:
                best, best_cost = pieces, cost
        return best

    def mlstm_scan(self, proj, q_col, k_col, v_col, gates, state, plan, heads, dim, vdim, floor, pieces=None):
        """The recurrence of parts/mlstm.py over the step's sequences: q, k (heads x dim) and v (heads x vdim) are
        columns of `proj`; state: {"S": [slots, heads, dim, vdim], "n": [slots, heads, dim], "m": [slots, heads]}
        float32 (advanced); float32 [T, heads * vdim]."""
        S, n, m = state["S"], state["n"], state["m"]
        if (S.dtype != torch.float32 or tuple(S.shape[1:]) != (heads, dim, vdim) or tuple(n.shape[1:]) != (heads, dim)
                or tuple(m.shape[1:]) != (heads,)):
            raise KernelError("mlstm_scan: the state is float32 S [slots, heads, dim, vdim], n [slots, heads, dim], m [slots, heads]")
        if gates.dtype != torch.float32 or tuple(gates.shape) != (plan.T, 2 * heads):
            raise KernelError("mlstm_scan: float32 log gates [T, 2 * heads]")
        if max(q_col, k_col) + heads * dim > proj.shape[1] or v_col + heads * vdim > proj.shape[1]:
            raise KernelError("mlstm_scan: the columns of q, k and v do not fit the rows")
        out = torch.empty((plan.T, heads * vdim), dtype=torch.float32, device=proj.device)
        longest = max(int(plan.max_new), 1)
        if pieces is None:
            cols = -(-vdim // 8) * 8 if vdim <= 64 else 64            # (the kernel's columns a block)
            # (blocks of nine warps: two on an SM up to a key size of 128, one above)
            pieces = self._pieces(longest, plan.n * heads * -(-vdim // cols), resident=self.sms * (2 if dim <= 128 else 1))
        piece = -(-longest // pieces)
        scratch = None
        if pieces > 1:
            scratch = torch.empty(self.lib.ember_mlstm_scan_scratch(plan.n, pieces, heads, dim, vdim), dtype=torch.float32,
                                  device=proj.device)
        self._call("ember_mlstm_scan", proj.data_ptr(), proj.stride(0), int(q_col), int(k_col), int(v_col), gates.data_ptr(),
                   S.data_ptr(), n.data_ptr(), m.data_ptr(), out.data_ptr(), plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(),
                   plan.cu_new.data_ptr(), plan.n, heads, dim, vdim, float(floor), piece, pieces, self._ptr(scratch),
                   _code(proj.dtype))
        if pieces > 1:
            self.launches += 2
        return out

    def mingru(self, proj, z_col, x_col, g_col, bias_z, bias_x, state, plan, width, out_dtype, pieces=None):
        """The recurrence of parts/mingru.py over the step's sequences: the gate's, the candidate's and the output gate's
        columns of `proj`; state float32 [slots, width] (advanced); S_t * silu(g_t) as [T, width] of `out_dtype`."""
        if state.dtype != torch.float32 or tuple(state.shape[1:]) != (width,):
            raise KernelError("mingru: the state is float32 [slots, width]")
        if max(z_col, x_col, g_col) + width > proj.shape[1]:
            raise KernelError("mingru: the columns do not fit the rows")
        out = torch.empty((plan.T, width), dtype=out_dtype, device=proj.device)
        longest = max(int(plan.max_new), 1)
        if pieces is None:
            pieces = self._pieces(longest, plan.n * -(-width // 128))
        piece = -(-longest // pieces)
        scratch = None
        if pieces > 1:
            scratch = torch.empty(self.lib.ember_mingru_scratch(plan.n, pieces, width), dtype=torch.float32, device=proj.device)
        self._call("ember_mingru", proj.data_ptr(), proj.stride(0), int(z_col), int(x_col), int(g_col), bias_z.data_ptr(),
                   bias_x.data_ptr(), state.data_ptr(), out.data_ptr(), plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(),
                   plan.cu_new.data_ptr(), plan.n, width, piece, pieces, self._ptr(scratch), _code(proj.dtype), _code(out_dtype))
        if pieces > 1:
            self.launches += 2
        return out

    # ------------------------------------------------------------------ a table of token pairs
    def pair_table_add(self, x, plan, table, state, mul_prev, mul_cur, buckets):
        """x[t] += table[row] in place, row = (token before * mul_prev + token * mul_cur) mod buckets, or the table's
        last row for a sequence's first token; state int32 [slots, 1]: each sequence's last token so far (advanced)."""
        T, d = x.shape
        if x.dtype != torch.float32 or table.shape != (buckets + 1, d) or state.dtype != torch.int32:
            raise KernelError("pair_table_add: a float32 stream, a table of buckets + 1 rows of its width, int32 state")
        self._call("ember_pair_table_add", self._dense(x, "stream").data_ptr(), plan.tokens.data_ptr(), plan.positions.data_ptr(),
                   plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(), plan.cu_new.data_ptr(),
                   self._dense(table, "pair table").data_ptr(), self._dense(state, "state").data_ptr(), T, d, int(mul_prev),
                   int(mul_cur), int(buckets), 1 << 30, _code(table.dtype))
        return x

    # ------------------------------------------------------------------ rotation, rows of low rank, products per head
    def rotate(self, src, dst, positions, heads, src_col, src_head, dst_col, dst_head, width, freqs, magnitude, dims,
               interleaved=False):
        """For every token t and head h < heads: `width` values from column src_col + h * src_head of src, their first
        `dims` rotated by the token's position (pair i with i + dims / 2, angle position * freqs[i], cos and sin times
        `magnitude`), written to column dst_col + h * dst_head of dst.  src and dst may be one tensor.  `interleaved`:
        pair i is dimensions 2i and 2i + 1."""
        T = src.shape[0]
        if src.stride(1) != 1 or dst.stride(1) != 1 or dst.shape[0] != T or freqs.dtype != torch.float32 or freqs.numel() != dims // 2:
            raise KernelError("rotate: rows of contiguous values, a float32 frequency for every pair")
        if src_col + (heads - 1) * src_head + width > src.shape[1] or dst_col + (heads - 1) * dst_head + width > dst.shape[1]:
            raise KernelError("rotate: the heads do not fit the rows")
        self._call("ember_rotate_pairs", src.data_ptr(), src.stride(0), int(src_col), int(src_head), _code(src.dtype), dst.data_ptr(),
                   dst.stride(0), int(dst_col), int(dst_head), _code(dst.dtype), T, int(heads), int(width),
                   positions.data_ptr(), freqs.data_ptr(), float(magnitude), int(dims), 1 if interleaved else 0)
        return dst

    def latent_rows(self, down, plan, q_rank, q_norm, kv_norm, kv_rank, rot_dim, eps, rotary, cache, out_dtype):
        """From float32 rows [T, q_rank (| kv_rank | rot_dim)]: the RMS-normed query row (returned, `out_dtype`), and with
        a cache the RMS-normed row c and the rotated key part, written at each token's position into the cache's key
        and value pages."""
        T, width = down.shape
        if down.dtype != torch.float32 or q_norm.shape[0] != q_rank:
            raise KernelError("latent_rows: float32 rows and a gain of the query row's width")
        c_q = torch.empty((T, q_rank), dtype=out_dtype, device=down.device)
        if cache is not None:
            if cache.k.dtype != out_dtype or tuple(cache.k.shape[1:]) != (1, 64, kv_rank) or tuple(cache.v.shape[1:]) != (1, 64, rot_dim):
                raise KernelError("latent_rows: the cache's pages do not have the mixer's row sizes or element type")
            if kv_norm.shape[0] != kv_rank:
                raise KernelError("latent_rows: a gain of the cached row's width")
        pages = None if cache is None else plan.pages[cache.group_index]
        self._call("ember_latent_rows", self._dense(down, "rows").data_ptr(), width, int(q_rank), q_norm.data_ptr(),
                   self._ptr(kv_norm), int(kv_rank), int(rot_dim), float(eps), rotary.freqs.data_ptr(), float(rotary.magnitude),
                   int(rotary.dims), c_q.data_ptr(), None if cache is None else cache.k.data_ptr(),
                   None if cache is None else cache.v.data_ptr(), plan.positions.data_ptr(), plan.token_seq.data_ptr(),
                   plan.seq_slot.data_ptr(), self._ptr(pages), plan.max_blocks, T, _code(out_dtype))
        return c_q

    def head_linear(self, a, a_col, a_head, w, out, out_col, out_head):
        """out[t, out_col + h * out_head + (0..N)] = a[t, a_col + h * a_head + (0..K)] w[h]^T for every head h of
        w [heads, N, K]; float32 sums."""
        heads, N, K = w.shape
        T = a.shape[0]
        if a.dtype != w.dtype or out.dtype != w.dtype or out.shape[0] != T or a.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("head_linear: rows, matrices and output of one element type")
        if a_col + (heads - 1) * a_head + K > a.shape[1] or out_col + (heads - 1) * out_head + N > out.shape[1]:
            raise KernelError("head_linear: the heads do not fit the rows")
        if w.dtype == torch.bfloat16 and T > SMALL_M and self.gemm == "lt":
            # the library's strided batch (a head's offset as the batch stride), where everything lies on 16 bytes
            ws = self._lt_workspace()
            rc = self._call("ember_head_linear_bf16", a.data_ptr() + 2 * int(a_col), a.stride(0), int(a_head),
                            self._dense(w, "matrices").data_ptr(), out.data_ptr() + 2 * int(out_col), out.stride(0), int(out_head),
                            T, heads, N, K, ws.data_ptr(), ws.numel(), allow=(2,))
            if rc == 0:
                return out
        self._call("ember_head_linear", a.data_ptr(), a.stride(0), int(a_col), int(a_head), self._dense(w, "matrices").data_ptr(),
                   out.data_ptr(), out.stride(0), int(out_col), int(out_head), T, heads, N, K, _code(w.dtype))
        return out

    def latent_attention(self, rows, cache, plan, heads, kv_rank, rot_dim, scale, out_dtype):
        """Causal attention of the step's query heads (each `kv_rank` values for the cached rows, then `rot_dim` for the
        shared key part) over the cache; per head the weighted sum of the cached rows: [T, heads * kv_rank]."""
        T = rows.shape[0]
        if rows.dtype != cache.k.dtype or out_dtype != rows.dtype or rows.shape[1] != heads * (kv_rank + rot_dim):
            raise KernelError("latent_attention: query rows, cache and output of one element type and fitting sizes")
        if tuple(cache.k.shape[1:]) != (1, 64, kv_rank) or tuple(cache.v.shape[1:]) != (1, 64, rot_dim):
            raise KernelError("latent_attention: the cache's pages do not have the mixer's row sizes")
        out = torch.empty((T, heads * kv_rank), dtype=out_dtype, device=rows.device)
        pages = plan.pages[cache.group_index]
        if self.latent_fast and rows.dtype == torch.bfloat16:
            # one token each: the pages in chunks, a block a chunk, so that the launch fills the chip about twice
            blocks = min(plan.max_blocks, max(1, -(-plan.max_end // 64)))
            n_chunks, per_chunk = 1, plan.max_blocks
            if plan.all_single and plan.T == plan.n:
                tiles = plan.n * -(-heads // 64)
                n_chunks = max(1, min(blocks, 2 * self.sms // max(tiles, 1)))
                per_chunk = self.latent_pages_per_chunk or -(-blocks // n_chunks)
                n_chunks = -(-blocks // per_chunk)
            n_scratch = self.lib.ember_latent_attention_mma_scratch(T * heads, kv_rank, n_chunks)
            scratch = torch.empty(n_scratch, dtype=torch.float32, device=rows.device) if n_scratch else None
            rc = self._call("ember_latent_attention_mma", self._dense(rows, "query rows").data_ptr(), cache.k.data_ptr(),
                            cache.v.data_ptr(), out.data_ptr(), self._ptr(scratch), plan.seq_slot.data_ptr(),
                            plan.seq_start.data_ptr(), plan.cu_new.data_ptr(), pages.data_ptr(), plan.max_blocks, plan.n,
                            max(int(plan.max_new), 1), T, heads, kv_rank, rot_dim, float(scale), n_chunks, per_chunk, allow=(2,))
            if rc == 0:
                self.launches += 1 if n_chunks > 1 else 0      # (the merge)
                return out
        self._call("ember_latent_attention_plain", self._dense(rows, "query rows").data_ptr(), cache.k.data_ptr(),
                   cache.v.data_ptr(), out.data_ptr(), plan.positions.data_ptr(), plan.token_seq.data_ptr(),
                   plan.seq_slot.data_ptr(), pages.data_ptr(), plan.max_blocks, T, heads, kv_rank, rot_dim, float(scale),
                   _code(rows.dtype))
        return out

    # ------------------------------------------------------------------ gated delta rule
    DELTA_CHUNKS_FROM = 64   # new tokens of a step's longest sequence from which the delta rule runs in chunks (bfloat16)

    def delta_rule(self, qkv, proj, b_col, a_col, a_log, dt_bias, state, plan, heads, kv_heads, dim, vdim, unit_eps,
                   chunked=None):
        """The recurrence of parts/delta.py over the step's sequences: qkv [T, q | k | v] (the convolution's output),
        the raw beta and step in `heads` columns each from b_col and a_col of `proj`, state float32
        [slots, heads, dim, vdim] (advanced); float32 o [T, heads * vdim].  chunked: the closed form over chunks of 64
        tokens (prompts; None lets the step's shape and the element type decide: bfloat16 steps with a sequence of
        DELTA_CHUNKS_FROM new tokens or more, key sizes that are multiples of 4 up to 128); else token by token, the
        sums in one fixed order (the 32-bit path, one-token steps)."""
        T = qkv.shape[0]
        if qkv.shape[1] != 2 * kv_heads * dim + heads * vdim or qkv.dtype != proj.dtype:
            raise KernelError("delta_rule: rows of q | k | v in the projection's element type")
        if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, dim, vdim):
            raise KernelError("delta_rule: the state is float32 [slots, heads, dim, vdim]")
        self._dense(qkv, "q | k | v")
        out = torch.empty((T, heads * vdim), dtype=torch.float32, device=qkv.device)
        if chunked is None:
            chunked = qkv.dtype == torch.bfloat16 and plan.max_new >= self.DELTA_CHUNKS_FROM
        chunked = bool(chunked) and dim % 4 == 0 and dim <= 128
        slots = (T // 64 + plan.n) if chunked else 0        # chunks are numbered through the sequences: at most this many
        scratch = torch.empty(self.lib.ember_delta_rule_scratch(T, heads, kv_heads, dim, vdim, slots), dtype=torch.float32,
                              device=qkv.device)
        self._call("ember_delta_rule", qkv.data_ptr(), proj.data_ptr(), proj.stride(0), int(b_col), int(a_col), a_log.data_ptr(),
                   dt_bias.data_ptr(), state.data_ptr(), out.data_ptr(), scratch.data_ptr(), plan.seq_slot.data_ptr(),
                   plan.seq_start.data_ptr(), plan.cu_new.data_ptr(), T, plan.n, heads, kv_heads, dim, vdim, float(unit_eps),
                   max(int(plan.max_new), 1), slots, _code(qkv.dtype))
        self.launches += 2 if chunked else 1      # (the prepare kernel, the chunks' factors)
        return out

    # ------------------------------------------------------------------ token shift, per-layer token input
    def token_shift(self, h, mu, state, plan):
        """h[t] + (h[t-1] - h[t]) * mu per sequence of the step, the row before a sequence's first token of the step being
        state[slot] (zeros at position 0); state [slots, width] float32 then holds each sequence's last row."""
        T, width = h.shape
        if mu.dtype != torch.float32 or mu.numel() != width or state.dtype != torch.float32 or state.shape[1] != width:
            raise KernelError("token_shift: a float32 blend vector and float32 state rows of the rows' width")
        out = torch.empty_like(h)
        self._call("ember_token_shift", self._dense(h, "rows").data_ptr(), out.data_ptr(), mu.data_ptr(), state.data_ptr(),
                   plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(), plan.cu_new.data_ptr(), T, width,
                   _code(h.dtype))
        return out

    def side_input(self, x, plan, table, col, dim, w_gate, w_proj, w_norm, eps):
        """x += unit_rms(W_proj (gelu_tanh(W_gate x) * e)) * w_norm in place, e = `dim` columns from `col` of each token's
        row of `table`: the stream's rows in the compute type, the first product with its GELU, the table's values, the
        second product with float32 sums, and the norm with the sum (`add_normed`)."""
        T, width = x.shape
        dtype = w_gate.dtype
        if x.dtype != torch.float32 or table.dtype != dtype or w_proj.dtype != dtype or \
                tuple(w_gate.shape) != (dim, width) or tuple(w_proj.shape) != (width, dim) or w_norm.numel() != width:
            raise KernelError("side_input: a float32 stream, the table and both matrices of one element type and fitting sizes")
        rows = self._dense(x, "stream")
        if dtype != torch.float32:
            rows = torch.empty((T, width), dtype=dtype, device=x.device)
            self._call("ember_cast_rows", x.data_ptr(), rows.data_ptr(), T * width, _code(dtype))
        z = self.linear(rows, w_gate, None, act="gelu_tanh", out_dtype=dtype)
        g = torch.empty_like(z)
        self._call("ember_table_gate", z.data_ptr(), g.data_ptr(), plan.tokens.data_ptr(), table.data_ptr(), table.shape[0],
                   table.shape[1], int(col), int(dim), T, _code(dtype))
        y = self.linear(g, w_proj, None, out_dtype=torch.float32)
        return self.add_normed(x, [(y, 1.0)], w_norm, eps)

    # ------------------------------------------------------------------ linear attention, the generalized delta rule
    def low_rank_out(self, proj, col, w2, bias, act):
        """bias + act(proj[:, col : col + rank]) W2^T with float32 sums: the second half of a product of low rank;
        w2 float32 [rank, n_out] (W2 transposed: the kernel reads an output's weights across its rows), act "none" or
        "tanh".  float32 [T, n_out]."""
        rank, n_out = w2.shape
        if act not in ("none", "tanh") or w2.dtype != torch.float32 or bias.dtype != torch.float32 or bias.numel() != n_out \
                or col + rank > proj.shape[1] or proj.stride(1) != 1:
            raise KernelError("low_rank_out: float32 [rank, outputs] and bias, the rank's columns inside the rows")
        out = torch.empty((proj.shape[0], n_out), dtype=torch.float32, device=proj.device)
        self._call("ember_low_rank_out", proj.data_ptr(), proj.stride(0), int(col), rank, self._dense(w2, "w2").data_ptr(), bias.data_ptr(),
                   out.data_ptr(), proj.shape[0], n_out, 1 if act == "tanh" else 0, _code(proj.dtype))
        return out

    RECURRENCE_PIECES_FROM = 256    # new tokens of a step's longest sequence from which a recurrence is walked in pieces

    def _recurrence_pieces(self, rule, plan, heads, dim, vdim, pieces, device):
        """(count of pieces, scratch) for a walk of gated linear attention (rule 0) or the generalized delta rule (1):
        sequences that bring many tokens are cut into pieces that are walked side by side.  pieces: None chooses, 0
        forces one walk, a count forces pieces (the tests')."""
        if pieces is None:
            pieces = 0 if plan.all_single or plan.max_new < self.RECURRENCE_PIECES_FROM else 1
        if not pieces:
            return 0, None
        count = -(-max(int(plan.max_new), 1) // self.lib.ember_recurrence_piece())
        floats = self.lib.ember_recurrence_scratch(rule, plan.n, count, heads, dim, vdim)
        return count, torch.empty(floats, dtype=torch.float32, device=device)

    def gla_scan(self, proj, q_col, k_col, v_col, z, tau, state, plan, heads, dim, vdim, pieces=None):
        """Gated linear attention token by token: S <- diag(sigmoid(z)^(1/tau)) S + k v^T, o = S^T (q dim^(-1/2)); q, k, v
        from columns of `proj`, z float32 [T, heads * dim], state float32 [slots, heads, dim, vdim].  float32 [T, heads * vdim]."""
        T = proj.shape[0]
        if z.dtype != torch.float32 or tuple(z.shape) != (T, heads * dim) or state.dtype != torch.float32 or \
                tuple(state.shape[1:]) != (heads, dim, vdim) or proj.stride(1) != 1:
            raise KernelError("gla_scan: float32 decays [T, heads * dim] and state [slots, heads, dim, vdim]")
        out = torch.empty((T, heads * vdim), dtype=torch.float32, device=proj.device)
        count, scratch = self._recurrence_pieces(0, plan, heads, dim, vdim, pieces, proj.device)
        self._call("ember_gla_scan", proj.data_ptr(), proj.stride(0), int(q_col), int(k_col), int(v_col), self._dense(z, "z").data_ptr(),
                   float(tau), state.data_ptr(), out.data_ptr(), plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(),
                   plan.cu_new.data_ptr(), plan.n, heads, dim, vdim, count, self._ptr(scratch), _code(proj.dtype))
        self.launches += 2 if count else 0       # (the carry kernel and the second walk)
        return out

    def generalized_delta_rule(self, proj, r_col, k_col, v_col, a_col, a_bias, wz, decay_coef, state, plan, heads, dim, unit_eps,
                               pieces=None):
        """S <- diag(w) S - (a u)(u^T S) + k v^T, o = S^T r, with w = exp(-decay_coef * sigmoid(wz)), a = sigmoid(a_in +
        a_bias), u the unit key; r, k, v, a_in from columns of `proj`, wz float32 [T, heads * dim], state float32
        [slots, heads, dim, dim].  float32 [T, heads * dim]."""
        T, m = proj.shape[0], heads * dim
        if wz.dtype != torch.float32 or tuple(wz.shape) != (T, m) or state.dtype != torch.float32 or a_bias.numel() != m or \
                tuple(state.shape[1:]) != (heads, dim, dim) or proj.stride(1) != 1:
            raise KernelError("generalized_delta_rule: float32 decays [T, heads * dim] and state [slots, heads, dim, dim]")
        out = torch.empty((T, m), dtype=torch.float32, device=proj.device)
        count, scratch = self._recurrence_pieces(1, plan, heads, dim, dim, pieces, proj.device)
        self._call("ember_generalized_delta_rule", proj.data_ptr(), proj.stride(0), int(r_col), int(k_col), int(v_col), int(a_col),
                   a_bias.data_ptr(), self._dense(wz, "decays").data_ptr(), float(decay_coef), float(unit_eps), state.data_ptr(),
                   out.data_ptr(), plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(), plan.cu_new.data_ptr(), plan.n, heads, dim,
                   count, self._ptr(scratch), _code(proj.dtype))
        self.launches += 2 if count else 0
        return out

    # ------------------------------------------------------------------ experts by table
    def moe_route(self, tokens, T, table, experts, top):
        """The step's (token, choice) pairs by expert: (expert of each pair, running counts, pairs in expert order).
        tokens None: row t of `table` [T, top] is token t's choice (what `moe_pick` made)."""
        pairs = T * top
        buf = torch.empty(2 * pairs + experts + 1, dtype=torch.int32, device=table.device)
        pair_expert, offsets, order = buf[:pairs], buf[pairs:pairs + experts + 1], buf[pairs + experts + 1:]
        self._call("ember_moe_route", self._ptr(tokens), table.data_ptr(), T, top, experts, table.shape[0],
                   pair_expert.data_ptr(), offsets.data_ptr(), order.data_ptr())
        return pair_expert, offsets, order, T, top, experts

    def _moe_tiled(self, pairs, dtype, tiled, k, n_out):
        """Tiles from MOE_TILE_PAIRS pairs on in bfloat16, where rows are whole 16-byte pieces and outputs come in twos."""
        if tiled is None:
            tiled = dtype == torch.bfloat16 and pairs >= MOE_TILE_PAIRS
        return 1 if tiled and k % 8 == 0 and n_out % 2 == 0 else 0

    def moe_pick(self, logits, correction, experts, top, groups, keep_groups, route_scale):
        """The router's choice for every row of float32 logits [T, >= experts]: scores sigmoid(z); chosen on score +
        correction among the experts of the `keep_groups` groups (of `groups` equal groups of neighbours) whose two
        largest choice scores add up to the most; weights = the chosen's scores over their sum (+ 1e-20) times
        `route_scale`.  Returns (chosen int32 [T, top], weights float32 [T, top])."""
        T = logits.shape[0]
        if logits.dtype != torch.float32 or logits.shape[1] < experts or correction.dtype != torch.float32 or correction.numel() != experts:
            raise KernelError("moe_pick: float32 logits of at least `experts` columns and a float32 correction an expert")
        chosen = torch.empty((T, top), dtype=torch.int32, device=logits.device)
        weights = torch.empty((T, top), dtype=torch.float32, device=logits.device)
        self._call("ember_moe_pick", self._dense(logits, "logits").data_ptr(), logits.shape[1], correction.data_ptr(), T, int(experts),
                   int(top), int(groups), int(keep_groups), float(route_scale), chosen.data_ptr(), weights.data_ptr())
        return chosen, weights

    def moe_combine(self, x, y, weights, shared, logits, gate_col):
        """x + sum_k weights[:, k] * y[:, k, :] (+ shared, times sigmoid(logits[:, gate_col]) where logits are given),
        float32, as a new tensor."""
        T, top, width = y.shape
        if any(t is not None and t.dtype != torch.float32 for t in (x, y, weights, shared, logits)) or tuple(x.shape) != (T, width) \
                or tuple(weights.shape) != (T, top) or (shared is not None and tuple(shared.shape) != (T, width)):
            raise KernelError("moe_combine: float32 rows of fitting sizes")
        out = torch.empty_like(x)
        self._call("ember_moe_combine", self._dense(x, "stream").data_ptr(), self._dense(y, "experts' rows").data_ptr(),
                   self._dense(weights, "weights").data_ptr(), self._ptr(None if shared is None else self._dense(shared, "shared rows")),
                   self._ptr(logits), 0 if logits is None else logits.shape[1], int(gate_col), out.data_ptr(), T, top, width)
        return out

    def moe_gate_up(self, h, w_gate_up, routing, out_dtype, tiled=None, limit=0.0, alpha=1.0, shift=0.0):
        pair_expert, offsets, order, T, top, experts = routing
        inner, width = w_gate_up.shape[1] // 2, w_gate_up.shape[2]
        if h.dtype != w_gate_up.dtype or out_dtype != h.dtype or h.shape[1] != width or w_gate_up.shape[0] != experts:
            raise KernelError("moe_gate_up: rows, stacked matrices and output of one element type and fitting sizes")
        out = torch.empty((T * top, inner), dtype=out_dtype, device=h.device)
        self._call("ember_moe_gate_up_act", self._dense(h, "rows").data_ptr(), self._dense(w_gate_up, "experts").data_ptr(),
                   pair_expert.data_ptr(), offsets.data_ptr(), order.data_ptr(), out.data_ptr(), T, top, experts, width,
                   inner, self._moe_tiled(T * top, h.dtype, tiled, width, inner), _code(h.dtype), float(limit), float(alpha),
                   float(shift))
        return out

    def moe_down(self, inner_rows, w_down, routing, tiled=None):
        pair_expert, offsets, order, T, top, experts = routing
        width, inner = w_down.shape[1], w_down.shape[2]
        if inner_rows.dtype != w_down.dtype or tuple(inner_rows.shape) != (T * top, inner) or w_down.shape[0] != experts:
            raise KernelError("moe_down: rows and stacked matrices of one element type and fitting sizes")
        out = torch.empty((T, top, width), dtype=torch.float32, device=inner_rows.device)
        self._call("ember_moe_down", self._dense(inner_rows, "rows").data_ptr(), self._dense(w_down, "experts").data_ptr(),
                   pair_expert.data_ptr(), offsets.data_ptr(), order.data_ptr(), out.data_ptr(), T, top, experts, width,
                   inner, self._moe_tiled(T * top, inner_rows.dtype, tiled, inner, width), _code(inner_rows.dtype))
        return out

    # ------------------------------------------------------------------ sampling
    sample_takes_base = True

    def sample(self, logits, temperature, top_k, top_p, seed, streams, counters, counter_base: int = 0, out=None):
        """One token per row of float32 logits.  `streams` and `counters` (int32, one per row) key
        the uniform number of each row's draw; `counter_base` is added to every row's counter.  `out`:
        where the ids go (int32, one per row; default: a new tensor)."""
        rows, V = logits.shape
        if logits.dtype != torch.float32:
            raise KernelError("sample: logits are float32")
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        elif out.dtype != torch.int32 or out.shape != (rows,) or not out.is_contiguous() or out.device != logits.device:
            raise KernelError("sample: the ids go into a contiguous int32 tensor with one entry per row, on the logits' device")
        self._call("ember_sample", self._dense(logits, "logits").data_ptr(), out.data_ptr(), rows, V, float(temperature),
                   int(top_k), float(top_p), int(seed) & 0xFFFFFFFFFFFFFFFF, streams.data_ptr(), counters.data_ptr(),
                   int(counter_base))
        return out
