"""Mega-MoE entry points with the reference's Python surface (deep_gemm/mega/__init__.py:18-176):
``get_symm_buffer_for_mega_moe`` -> ``SymmBuffer`` (the caller copies x / x_sf / topk_idx / topk_weights into its
views), ``transform_weights_for_mega_moe`` and ``fp8_fp4_mega_moe``. The layer itself runs in libdgb200.so."""
import ctypes
import types
from typing import Optional, Tuple

import torch

from . import _lib
from .utils.math import align

_NUM_LAYOUT_WORDS = 16
_GATE_UP_INTERLEAVE = 128  # rows: [gate 0..127 | up 0..127 | gate 128..255 | ...]: an L1 output tile is 128 gate + 128 up channels


def get_token_alignment_for_mega_moe() -> int:
    """Reference: csrc/apis/mega.hpp:19-21."""
    return _lib.lib().dgb200_get_token_alignment_for_mega_moe()


def get_segment_alignment_for_mega_moe() -> int:
    """Rows each expert's segment is padded to in the layer's expert-sorted buffers (no reference counterpart)."""
    return _lib.lib().dgb200_get_segment_alignment_for_mega_moe()


def get_block_m_for_mega_moe(num_ranks: int, num_experts: int, num_max_tokens_per_rank: int, num_tokens: int,
                             num_topk: int, mma_type: str = 'fp8xfp4') -> int:
    """Rows of one M tile. The reference picks 16..192 by expected rows per expert (csrc/apis/mega.hpp:23-32);
    this kernel always tiles tokens by 128 and clips per expert."""
    del num_ranks, num_experts, num_max_tokens_per_rank, num_tokens, num_topk, mma_type
    return 128


_MMA_TYPES = ('fp8xfp4', 'nvfp4xnvfp4', 'bf16xbf16')


def _buffer_layout(num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
                   mma_type='fp8xfp4', shared_intermediate_hidden=0):
    words = (ctypes.c_int64 * 26)()
    if mma_type == 'fp8xfp4':
        _lib.check(_lib.lib().dgb200_get_symm_buffer_layout_for_mega_moe_ex(
            num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
            shared_intermediate_hidden, ctypes.cast(words, ctypes.c_void_p)))
    elif mma_type == 'bf16xbf16':
        _lib.check(_lib.lib().dgb200_get_symm_buffer_layout_for_bf16_mega_moe(
            num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
            shared_intermediate_hidden, ctypes.cast(words, ctypes.c_void_p)))
    else:
        _lib.check(_lib.lib().dgb200_get_symm_buffer_layout_for_nvfp4_mega_moe(
            num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
            ctypes.cast(words, ctypes.c_void_p)))
    keys = ['total', 'x', 'x_sf', 'topk_idx', 'topk_weights', 'l1_acts', 'l1_sf', 'l2_acts', 'l2_sf', 'max_rows',
            'dest_row', 'src_of_row', 'expert_start', 'expert_end', 'l2_out', 'row_weight',
            'shared_x_sf', 'shared_l2_acts', 'shared_l2_sf', 'shared_out', 'flags',
            'my_base', 'my_dest', 'my_slot', 'guest_expert', 'rank_rows']
    return dict(zip(keys, list(words)))


class SymmBuffer:
    """One flat buffer per rank: caller-written inputs first, the layer's private workspace after them.
    Reference: SymmBuffer, deep_gemm/mega/__init__.py:18-66."""

    def __init__(self, group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                 intermediate_hidden: int, num_shared_experts: int = 0, mma_type: str = 'fp8xfp4',
                 activation: str = 'swiglu'):
        if activation != 'swiglu':
            raise RuntimeError(f'Only `swiglu` activation is supported, got `{activation}`')
        if mma_type not in _MMA_TYPES:
            raise RuntimeError(f'MMA type must be one of {_MMA_TYPES}, got `{mma_type}`')
        if num_shared_experts < 0 or (num_shared_experts > 0 and mma_type not in ('fp8xfp4', 'bf16xbf16')):
            raise RuntimeError('shared experts need num_shared_experts >= 0 and the `fp8xfp4` or `bf16xbf16` MMA type')
        self.num_shared_experts = num_shared_experts
        self.group = group
        self.num_ranks = 1 if group is None else group.size()
        self.rank = 0 if group is None else group.rank()
        self.num_experts, self.num_topk = num_experts, num_topk
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.hidden, self.intermediate_hidden = hidden, intermediate_hidden
        self.mma_type = mma_type
        self.layout = _buffer_layout(self.num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden,
                                     intermediate_hidden, mma_type, intermediate_hidden * num_shared_experts)
        num_bytes = self.layout['total']
        if self.num_ranks == 1:
            self.buffer = torch.empty(num_bytes, dtype=torch.int8, device='cuda')
            self.handle = types.SimpleNamespace(buffer_ptrs=[self.buffer.data_ptr()])
        else:
            import torch.distributed._symmetric_memory as symm_mem
            self.buffer = symm_mem.empty(num_bytes, dtype=torch.int8, device='cuda')
            self.handle = symm_mem.rendezvous(self.buffer, group=group)
        self.buffer.zero_()
        if group is not None:
            group.barrier()
        torch.cuda.synchronize()

        t, lay = num_max_tokens_per_rank, self.layout
        def view(offset, nbytes, dtype, shape):
            return self.buffer[offset:offset + nbytes].view(dtype).view(shape)
        if mma_type == 'fp8xfp4':
            self.x = view(lay['x'], t * hidden, torch.float8_e4m3fn, (t, hidden))
            self.x_sf = view(lay['x_sf'], t * (hidden // 128) * 4, torch.int32, (t, hidden // 128))
        elif mma_type == 'bf16xbf16':
            self.x = view(lay['x'], t * hidden * 2, torch.bfloat16, (t, hidden))
            self.x_sf = None
        else:  # packed E2M1 rows, four UE4M3 block scales (64 K elements) per int
            self.x = view(lay['x'], t * hidden // 2, torch.int8, (t, hidden // 2))
            self.x_sf = view(lay['x_sf'], t * (hidden // 64) * 4, torch.int32, (t, hidden // 64))
        self.topk_idx = view(lay['topk_idx'], t * num_topk * 8, torch.int64, (t, num_topk))
        self.topk_weights = view(lay['topk_weights'], t * num_topk * 4, torch.float32, (t, num_topk))

    def destroy(self):
        self.handle = self.buffer = self.group = None
        self.x = self.x_sf = self.topk_idx = self.topk_weights = None


def get_symm_buffer_for_mega_moe(group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                                 intermediate_hidden: int, num_shared_experts: int = 0,
                                 use_fp8_dispatch: Optional[bool] = None, mma_type: str = 'fp8xfp4',
                                 activation: str = 'swiglu') -> SymmBuffer:
    """Reference: get_symm_buffer_for_mega_moe, deep_gemm/mega/__init__.py:69-94. ``group`` may be None for a
    single process."""
    num_max_tokens_per_rank = align(num_max_tokens_per_rank, get_token_alignment_for_mega_moe())
    if use_fp8_dispatch is not None and use_fp8_dispatch != (mma_type.split('x')[0] == 'fp8'):
        raise RuntimeError('use_fp8_dispatch contradicts mma_type')
    return SymmBuffer(group, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
                      num_shared_experts, mma_type=mma_type, activation=activation)


def _interleave_rows(t: torch.Tensor, gran: int) -> torch.Tensor:
    """[G, N, ...] with rows [gate | up] -> blocks of `gran` gate rows followed by the matching up rows. Strides of
    the result equal those of the input (packed scale factors stay MN-major)."""
    n = t.shape[1]
    half = n // 2
    if half % gran != 0:
        raise RuntimeError(f'intermediate size {half} must be a multiple of {gran}')
    r = torch.arange(n, device=t.device)
    block, within = r // (2 * gran), r % (2 * gran)
    src = torch.where(within < gran, gran * block + within, half + gran * block + within - gran)
    out = torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=t.device)
    out.copy_(t.index_select(1, src))
    return out


def _sf_rows_to_cp_order(sf: torch.Tensor) -> torch.Tensor:
    """Packed MN-major scale factors [G, N, Kp]: store every aligned group of 128 rows in the order tcgen05.cp reads
    (row r of a group at position 4 (r % 32) + r / 32), so the kernel copies them from shared to tensor memory as
    they land. Strides are kept."""
    n = sf.shape[1]
    if n % 128 != 0:
        raise RuntimeError(f'weight rows ({n}) must be a multiple of 128')
    pos = torch.arange(n, device=sf.device)
    src = (pos // 128) * 128 + (pos % 4) * 32 + (pos % 128) // 4  # the row that lands at position `pos`
    out = torch.empty_strided(sf.shape, sf.stride(), dtype=sf.dtype, device=sf.device)
    out.copy_(sf.index_select(1, src))
    return out


def _to_weight_tiles(w: torch.Tensor, tile_rows: int) -> torch.Tensor:
    """Packed FP4 weights [E, N, K / 2] -> the same bytes as contiguous tiles of ``tile_rows`` rows x 128 K elements, in the
    order (expert, row block, K block): the storage dgb200_get_weight_tile_rows_for_mega_moe asks for. The tensor keeps
    its shape; only libdgb200.so interprets the bytes."""
    e, n, kb2 = w.shape
    if tile_rows <= 0:
        return w
    if n % tile_rows != 0 or kb2 % 64 != 0:
        raise RuntimeError(f'weight rows ({n}) must be a multiple of {tile_rows} and K a multiple of 128')
    return w.view(e, n // tile_rows, tile_rows, kb2 // 64, 64).permute(0, 1, 3, 2, 4).contiguous().view(e, n, kb2)


def transform_weights_for_mega_moe(l1_weights: Tuple[torch.Tensor, torch.Tensor],
                                   l2_weights: Tuple[torch.Tensor, torch.Tensor], activation: str = 'swiglu'):
    """Reorders the L1 weights (and their packed scale factors) so that every 256-row block holds 128 gate channels
    followed by their 128 up channels (one L1 output tile), and stores the scale factors of both layers in the row order
    tcgen05.cp consumes. The transformed tensors are opaque to the caller, as in the reference
    (transform_weights_for_mega_moe, deep_gemm/mega/__init__.py:131-149, which interleaves by 8 and pre-transposes
    scale factors for its own kernel)."""
    if activation != 'swiglu':
        raise RuntimeError(f'Only `swiglu` activation is supported, got `{activation}`')
    if not isinstance(l1_weights, tuple):  # BF16 weights: only the gate/up interleave
        if l1_weights.dtype != torch.bfloat16 or l2_weights.dtype != torch.bfloat16 or l1_weights.dim() not in (2, 3):
            raise RuntimeError('bare weight tensors must be bfloat16 [E, N, K] (or [N, K] for shared experts)')
        if l1_weights.dim() == 2:
            return _interleave_rows(l1_weights.unsqueeze(0), _GATE_UP_INTERLEAVE)[0].contiguous(), l2_weights
        return _interleave_rows(l1_weights, _GATE_UP_INTERLEAVE).contiguous(), l2_weights
    if l1_weights[0].dim() == 2:  # shared experts: one FP8 matrix per layer, same reordering
        t1, t2 = transform_weights_for_mega_moe(tuple(t.unsqueeze(0) for t in l1_weights),
                                                tuple(t.unsqueeze(0) for t in l2_weights), activation)
        return tuple(t[0] for t in t1), tuple(t[0] for t in t2)
    # NVFP4 weights carry a third element, the per-expert FP32 scales, which no reordering touches
    gran = _GATE_UP_INTERLEAVE
    if len(l1_weights) == 2 and l1_weights[0].dtype == torch.int8:  # the FP8 x MXFP4 layer's routed experts
        gran = _lib.lib().dgb200_get_gate_up_interleave_for_mega_moe()
    l1_sf = _sf_rows_to_cp_order(_interleave_rows(l1_weights[1], gran))
    l1_w, l2_w = _interleave_rows(l1_weights[0], gran), l2_weights[0]
    if len(l1_weights) == 2 and l1_w.dtype == torch.int8:
        tile_rows = _lib.lib().dgb200_get_weight_tile_rows_for_mega_moe()
        l1_w, l2_w = _to_weight_tiles(l1_w, tile_rows), _to_weight_tiles(l2_w, tile_rows)
    return (l1_w, l1_sf) + tuple(l1_weights[2:]), (l2_w, _sf_rows_to_cp_order(l2_weights[1])) + tuple(l2_weights[2:])


MAX_GUEST_EXPERTS = 8


class _SpillInfo:
    """What the layer call needs to let hot experts spill rows to other ranks: the number of guest slots and, for each
    of the four weight tensors, its address on every rank. Keeps the symmetric allocations alive."""

    def __init__(self, num_guest_experts, peer_ptrs, keep):
        self.num_guest_experts = num_guest_experts
        self.peer_ptrs = peer_ptrs  # four lists of num_ranks addresses: l1_w, l1_w_sf, l2_w, l2_w_sf
        self.keep = keep


def share_weights_for_mega_moe(group, l1_weights: Tuple[torch.Tensor, torch.Tensor],
                               l2_weights: Tuple[torch.Tensor, torch.Tensor], num_guest_experts: int = 4):
    """Expert-parallel runs with skewed routing: lets ranks compute rows of other ranks' hot experts (no reference
    counterpart; the reference keeps every expert's rows on its owner, so its step time follows the most loaded rank).

    Takes the FP8 x MXFP4 layer's routed weights as ``transform_weights_for_mega_moe`` returned them, moves them into
    symmetric memory with room for ``num_guest_experts`` more experts behind the rank's own, and returns the same
    ``(weights, scales)`` pairs (views of the first ``E_local`` experts). ``fp8_fp4_mega_moe`` recognises them: every call
    then derives, from the exchanged per-expert counts, which rows of which hot experts move to less loaded ranks, and
    those ranks fetch the experts' weights from the owners into their guest slots during the call. Outputs are the same
    bits as without it. Collective: every rank of ``group`` must call it with the same ``num_guest_experts``."""
    if group is None or group.size() == 1 or num_guest_experts <= 0:
        return l1_weights, l2_weights
    if num_guest_experts > MAX_GUEST_EXPERTS:
        raise RuntimeError(f'at most {MAX_GUEST_EXPERTS} guest experts')
    if len(l1_weights) != 2 or l1_weights[0].dtype != torch.int8:
        raise RuntimeError('only the FP8 x MXFP4 layer (packed int8 weights + packed UE8M0 scales) can share its weights')
    import torch.distributed._symmetric_memory as symm_mem
    shared, ptrs, keep = [], [], []
    for t in (l1_weights[0], l1_weights[1], l2_weights[0], l2_weights[1]):
        experts = t.shape[0]
        per_expert = t.stride(0) * t.element_size()  # bytes: both weights and MN-major packed scales are expert-major
        if per_expert % 16 != 0 or t.storage_offset() != 0:
            raise RuntimeError('weight tensors must start their storage and hold a multiple of 16 bytes per expert')
        flat = symm_mem.empty((experts + num_guest_experts) * per_expert, dtype=torch.int8, device=t.device)
        handle = symm_mem.rendezvous(flat, group=group)
        flat.zero_()
        view = flat[:experts * per_expert].view(t.dtype).as_strided(t.shape, t.stride())
        view.copy_(t)
        shared.append(view)
        ptrs.append([int(p) for p in handle.buffer_ptrs])
        keep.append((flat, handle))
    info = _SpillInfo(num_guest_experts, ptrs, keep)
    for view in shared:
        view._dgb200_spill = info
    torch.cuda.synchronize()
    group.barrier()
    return (shared[0], shared[1]), (shared[2], shared[3])


def _check_weight(w, sf, num_groups, n, k, name, k_per_int=128):
    if not (w.is_cuda and w.dtype == torch.int8 and w.is_contiguous() and tuple(w.shape) == (num_groups, n, k // 2)):
        raise RuntimeError(f'{name} must be a contiguous CUDA int8 tensor of shape {(num_groups, n, k // 2)}')
    if not (sf.dtype == torch.int32 and tuple(sf.shape) == (num_groups, n, k // k_per_int) and sf.stride(1) == 1 and
            sf.stride(2) == align(n, 4) and sf.stride(0) == sf.stride(2) * sf.shape[2]):
        raise RuntimeError(f'{name} scale factors must be packed int32 {(num_groups, n, k // k_per_int)}, MN-major '
                           '(use transform_sf_into_required_layout / pack_nvfp4_sf_mn_major)')


def _check_shared_weight(w, sf, n, k, name):
    if not (w.is_cuda and w.dtype == torch.float8_e4m3fn and w.is_contiguous() and tuple(w.shape) == (n, k)):
        raise RuntimeError(f'{name} must be a contiguous CUDA float8_e4m3fn tensor of shape {(n, k)}')
    if not (sf.dtype == torch.int32 and tuple(sf.shape) == (n, k // 128) and sf.stride(0) == 1 and sf.stride(1) == align(n, 4)):
        raise RuntimeError(f'{name} scale factors must be packed UE8M0 int32 {(n, k // 128)}, MN-major')


def _run_layer(y, l1_weights, l2_weights, b, shared_l1_weights, shared_l2_weights, stats, activation_clamp, fast_math,
               x=None, logits=None):
    """Common argument checks and the call into dgb200_fp8_fp4_mega_moe_ex."""
    if b.mma_type != 'fp8xfp4':
        raise RuntimeError(f'the buffer was created for `{b.mma_type}`')
    num_local = b.num_experts // b.num_ranks
    _check_weight(l1_weights[0], l1_weights[1], num_local, 2 * b.intermediate_hidden, b.hidden, 'l1_weights')
    _check_weight(l2_weights[0], l2_weights[1], num_local, b.hidden, b.intermediate_hidden, 'l2_weights')
    if (shared_l1_weights is None) != (shared_l2_weights is None):
        raise RuntimeError('shared_l1_weights and shared_l2_weights must be given together')
    shared_inter = 0
    if shared_l1_weights is not None:
        shared_inter = shared_l2_weights[0].size(1)
        if shared_inter != b.intermediate_hidden * b.num_shared_experts or shared_inter == 0:
            raise RuntimeError('the buffer was created for a different number of shared experts')
        _check_shared_weight(shared_l1_weights[0], shared_l1_weights[1], 2 * shared_inter, b.hidden, 'shared_l1_weights')
        _check_shared_weight(shared_l2_weights[0], shared_l2_weights[1], b.hidden, shared_inter, 'shared_l2_weights')
    if not (y.is_cuda and y.dtype == torch.bfloat16 and y.dim() == 2 and y.size(1) == b.hidden and y.is_contiguous()):
        raise RuntimeError('y must be a contiguous CUDA bfloat16 [num_tokens, hidden] tensor')
    if x is not None and not (x.is_cuda and x.dtype == torch.bfloat16 and tuple(x.shape) == tuple(y.shape) and x.stride(1) == 1):
        raise RuntimeError('x must be a CUDA bfloat16 [num_tokens, hidden] tensor with unit inner stride')
    if logits is not None and not (logits.is_cuda and logits.dtype == torch.float32 and logits.is_contiguous() and
                                   tuple(logits.shape) == (y.size(0), b.num_experts)):
        raise RuntimeError('logits must be a contiguous CUDA float32 [num_tokens, num_experts] tensor')
    if stats is not None and not (stats.dtype == torch.int32 and stats.numel() == num_local and stats.is_contiguous()):
        raise RuntimeError('cumulative_local_expert_recv_stats must be a contiguous int32 [num_local_experts] tensor')
    ptrs = (ctypes.c_uint64 * len(b.handle.buffer_ptrs))(*[int(p) for p in b.handle.buffer_ptrs])
    p = lambda t: t.data_ptr() if t is not None else None
    spill = getattr(l1_weights[0], '_dgb200_spill', None) if b.num_ranks > 1 else None
    if spill is not None and any(getattr(t, '_dgb200_spill', None) is not spill for t in (l1_weights[1], l2_weights[0], l2_weights[1])):
        raise RuntimeError('l1_weights and l2_weights must come from the same share_weights_for_mega_moe call')
    peer_w = [(ctypes.c_uint64 * b.num_ranks)(*spill.peer_ptrs[i]) for i in range(4)] if spill is not None else [None] * 4
    args = _lib.MegaMoeArgs(
        struct_size=ctypes.sizeof(_lib.MegaMoeArgs), y=p(y), l1_w=p(l1_weights[0]), l1_w_sf=p(l1_weights[1]),
        l2_w=p(l2_weights[0]), l2_w_sf=p(l2_weights[1]),
        shared_l1_w=p(shared_l1_weights[0]) if shared_inter else None, shared_l1_w_sf=p(shared_l1_weights[1]) if shared_inter else None,
        shared_l2_w=p(shared_l2_weights[0]) if shared_inter else None, shared_l2_w_sf=p(shared_l2_weights[1]) if shared_inter else None,
        x_bf16=p(x), logits=p(logits), cumulative_local_expert_recv_stats=p(stats), buffer=p(b.buffer),
        peer_buffer_ptrs=ctypes.cast(ptrs, ctypes.c_void_p), x_bf16_row_stride=x.stride(0) if x is not None else 0,
        shared_intermediate_hidden=shared_inter, rank=b.rank, num_ranks=b.num_ranks, num_tokens=y.size(0),
        num_max_tokens_per_rank=b.num_max_tokens_per_rank, num_experts=b.num_experts, num_topk=b.num_topk, hidden=b.hidden,
        intermediate_hidden=b.intermediate_hidden,
        activation_clamp=float(activation_clamp) if activation_clamp is not None else 0.0, fast_math=int(fast_math),
        num_guest_experts=spill.num_guest_experts if spill is not None else 0,
        peer_l1_w=ctypes.cast(peer_w[0], ctypes.c_void_p) if spill is not None else None,
        peer_l1_w_sf=ctypes.cast(peer_w[1], ctypes.c_void_p) if spill is not None else None,
        peer_l2_w=ctypes.cast(peer_w[2], ctypes.c_void_p) if spill is not None else None,
        peer_l2_w_sf=ctypes.cast(peer_w[3], ctypes.c_void_p) if spill is not None else None)
    with torch.cuda.device(y.device):
        _lib.check(_lib.lib().dgb200_fp8_fp4_mega_moe_ex(ctypes.byref(args), _lib.current_stream_ptr()))


def fp8_fp4_mega_moe(y: torch.Tensor, l1_weights: Tuple[torch.Tensor, torch.Tensor],
                     l2_weights: Tuple[torch.Tensor, torch.Tensor], sym_buffer: SymmBuffer,
                     shared_l1_weights: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                     shared_l2_weights: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                     cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                     recipe: Tuple[int, int, int] = (1, 1, 32), activation: str = 'swiglu',
                     activation_clamp: Optional[float] = None, fast_math: bool = True) -> None:
    """y[t] = sum_k w[t,k] * Expert_{idx[t,k]}(x[t]) (+ SharedExperts(x[t])) over the inputs the caller placed in
    ``sym_buffer``. Shared experts: (float8_e4m3fn [2 * SI, H], packed UE8M0 int32 scales) and ([H, SI], scales), both
    passed through ``transform_weights_for_mega_moe``; the buffer must have been created with ``num_shared_experts``.
    Reference: fp8_fp4_mega_moe, deep_gemm/mega/__init__.py:153-176 and csrc/apis/mega.hpp:157-286."""
    if tuple(recipe) != (1, 1, 32):
        raise RuntimeError('recipe must be (1, 1, 32)')
    if activation != 'swiglu':
        raise RuntimeError('activation must be `swiglu`')
    _run_layer(y, l1_weights, l2_weights, sym_buffer, shared_l1_weights, shared_l2_weights,
               cumulative_local_expert_recv_stats, activation_clamp, fast_math)


def fp8_fp4_mega_moe_bf16_input(y: torch.Tensor, x: torch.Tensor, l1_weights: Tuple[torch.Tensor, torch.Tensor],
                                l2_weights: Tuple[torch.Tensor, torch.Tensor], sym_buffer: SymmBuffer,
                                logits: Optional[torch.Tensor] = None,
                                shared_l1_weights: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                                shared_l2_weights: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                                cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                                activation_clamp: Optional[float] = None, fast_math: bool = True) -> None:
    """``fp8_fp4_mega_moe`` with its prologue fused in (no reference counterpart: the reference's callers quantise x with
    per_token_cast_to_fp8 into the buffer and route with torch ops, README.md:72, tests/test_mega_moe.py:124-125).
    ``x`` is BF16 [num_tokens, hidden] and is quantised while it is dispatched; with ``logits`` the router fills the
    buffer's ``topk_idx`` / ``topk_weights`` first, otherwise the caller has. Same bits as the separate steps."""
    _run_layer(y, l1_weights, l2_weights, sym_buffer, shared_l1_weights, shared_l2_weights,
               cumulative_local_expert_recv_stats, activation_clamp, fast_math, x=x, logits=logits)


def nvfp4_mega_moe(y: torch.Tensor, l1_weights: Tuple[torch.Tensor, torch.Tensor, torch.Tensor],
                   l2_weights: Tuple[torch.Tensor, torch.Tensor, torch.Tensor], sym_buffer: SymmBuffer,
                   x_scale: torch.Tensor, act_scale: torch.Tensor,
                   cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                   activation_clamp: Optional[float] = None, fast_math: bool = True) -> None:
    """The layer of ``fp8_fp4_mega_moe`` with NVFP4 activations and weights (no reference counterpart).

    ``sym_buffer`` must have been created with ``mma_type='nvfp4xnvfp4'``; the caller writes packed E2M1 rows and
    their UE4M3 scales into ``x`` / ``x_sf`` (``per_token_cast_to_nvfp4_into``). Weights are
    (int8 [E, N, K / 2], packed MN-major int32 scales [E, N, K / 64], FP32 [E] tensor scales), L1 passed through
    ``transform_weights_for_mega_moe``. ``x_scale`` is the FP32 scalar x was quantised against and must be the same
    on every rank; ``act_scale`` is the calibrated FP32 scalar the post-SwiGLU activations are quantised against."""
    b = sym_buffer
    if b.mma_type != 'nvfp4xnvfp4':
        raise RuntimeError(f'the buffer was created for `{b.mma_type}`')
    num_local = b.num_experts // b.num_ranks
    _check_weight(l1_weights[0], l1_weights[1], num_local, 2 * b.intermediate_hidden, b.hidden, 'l1_weights', 64)
    _check_weight(l2_weights[0], l2_weights[1], num_local, b.hidden, b.intermediate_hidden, 'l2_weights', 64)
    for t, count, name in ((l1_weights[2], num_local, 'l1 tensor scales'), (l2_weights[2], num_local, 'l2 tensor scales'),
                           (x_scale, 1, 'x_scale'), (act_scale, 1, 'act_scale')):
        if not (t.is_cuda and t.dtype == torch.float32 and t.numel() == count and t.is_contiguous()):
            raise RuntimeError(f'{name} must be a contiguous CUDA float32 tensor of {count} element(s)')
    if not (y.is_cuda and y.dtype == torch.bfloat16 and y.dim() == 2 and y.size(1) == b.hidden and y.is_contiguous()):
        raise RuntimeError('y must be a contiguous CUDA bfloat16 [num_tokens, hidden] tensor')
    stats = cumulative_local_expert_recv_stats
    if stats is not None and not (stats.dtype == torch.int32 and stats.numel() == num_local and stats.is_contiguous()):
        raise RuntimeError('cumulative_local_expert_recv_stats must be a contiguous int32 [num_local_experts] tensor')
    ptrs = (ctypes.c_uint64 * len(b.handle.buffer_ptrs))(*[int(p) for p in b.handle.buffer_ptrs])
    p = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    with torch.cuda.device(y.device):
        _lib.check(_lib.lib().dgb200_nvfp4_mega_moe(
            p(y), p(l1_weights[0]), p(l1_weights[1]), p(l1_weights[2]), p(l2_weights[0]), p(l2_weights[1]),
            p(l2_weights[2]), p(x_scale), p(act_scale), p(stats), p(b.buffer), ctypes.cast(ptrs, ctypes.c_void_p),
            b.rank, b.num_ranks, y.size(0), b.num_max_tokens_per_rank, b.num_experts, b.num_topk, b.hidden,
            b.intermediate_hidden, float(activation_clamp) if activation_clamp is not None else 0.0, int(fast_math),
            _lib.current_stream_ptr()))


def nvfp4_mega_moe_bf16_input(y: torch.Tensor, x: torch.Tensor, l1_weights: Tuple[torch.Tensor, torch.Tensor, torch.Tensor],
                              l2_weights: Tuple[torch.Tensor, torch.Tensor, torch.Tensor], sym_buffer: SymmBuffer,
                              x_scale: torch.Tensor, act_scale: torch.Tensor, logits: Optional[torch.Tensor] = None,
                              cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                              activation_clamp: Optional[float] = None, fast_math: bool = True) -> None:
    """``nvfp4_mega_moe`` on a single rank with its prologue fused in (no reference counterpart): ``x`` is BF16
    [num_tokens, hidden] and is quantised to NVFP4 against ``x_scale`` while it is dispatched; with ``logits`` the router
    fills the buffer's ``topk_idx`` / ``topk_weights`` first, otherwise the caller has. Same bits as
    ``per_token_cast_to_nvfp4_into`` + ``route_sigmoid_topk`` + ``nvfp4_mega_moe``."""
    b = sym_buffer
    if b.mma_type != 'nvfp4xnvfp4' or b.num_ranks != 1:
        raise RuntimeError('needs a single-rank buffer created with mma_type=`nvfp4xnvfp4`')
    _check_weight(l1_weights[0], l1_weights[1], b.num_experts, 2 * b.intermediate_hidden, b.hidden, 'l1_weights', 64)
    _check_weight(l2_weights[0], l2_weights[1], b.num_experts, b.hidden, b.intermediate_hidden, 'l2_weights', 64)
    for t, count, name in ((l1_weights[2], b.num_experts, 'l1 tensor scales'), (l2_weights[2], b.num_experts, 'l2 tensor scales'),
                           (x_scale, 1, 'x_scale'), (act_scale, 1, 'act_scale')):
        if not (t.is_cuda and t.dtype == torch.float32 and t.numel() == count and t.is_contiguous()):
            raise RuntimeError(f'{name} must be a contiguous CUDA float32 tensor of {count} element(s)')
    if not (y.is_cuda and y.dtype == torch.bfloat16 and y.dim() == 2 and y.size(1) == b.hidden and y.is_contiguous()):
        raise RuntimeError('y must be a contiguous CUDA bfloat16 [num_tokens, hidden] tensor')
    if not (x.is_cuda and x.dtype == torch.bfloat16 and tuple(x.shape) == tuple(y.shape) and x.stride(1) == 1):
        raise RuntimeError('x must be a CUDA bfloat16 [num_tokens, hidden] tensor with unit inner stride')
    if logits is not None and not (logits.is_cuda and logits.dtype == torch.float32 and logits.is_contiguous() and
                                   tuple(logits.shape) == (y.size(0), b.num_experts)):
        raise RuntimeError('logits must be a contiguous CUDA float32 [num_tokens, num_experts] tensor')
    stats = cumulative_local_expert_recv_stats
    if stats is not None and not (stats.dtype == torch.int32 and stats.numel() == b.num_experts and stats.is_contiguous()):
        raise RuntimeError('cumulative_local_expert_recv_stats must be a contiguous int32 [num_experts] tensor')
    p = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    with torch.cuda.device(y.device):
        _lib.check(_lib.lib().dgb200_nvfp4_mega_moe_bf16_input(
            p(y), p(x), x.stride(0), p(logits), p(l1_weights[0]), p(l1_weights[1]), p(l1_weights[2]), p(l2_weights[0]),
            p(l2_weights[1]), p(l2_weights[2]), p(x_scale), p(act_scale), p(stats), p(b.buffer), y.size(0),
            b.num_max_tokens_per_rank, b.num_experts, b.num_topk, b.hidden, b.intermediate_hidden,
            float(activation_clamp) if activation_clamp is not None else 0.0, int(fast_math), _lib.current_stream_ptr()))


def bf16_mega_moe(y: torch.Tensor, l1_weights: torch.Tensor, l2_weights: torch.Tensor, sym_buffer: SymmBuffer,
                  shared_l1_weights: Optional[torch.Tensor] = None, shared_l2_weights: Optional[torch.Tensor] = None,
                  cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None, activation: str = 'swiglu',
                  activation_clamp: Optional[float] = None, fast_math: bool = True) -> None:
    """The layer with BF16 activations and weights. Reference: bf16_mega_moe, deep_gemm/mega/__init__.py:178-204.

    ``sym_buffer`` must have been created with ``mma_type='bf16xbf16'``; the caller writes ``x`` (bfloat16), ``topk_idx``
    and ``topk_weights``. Weights are bfloat16 [E_local, 2 * inter, hidden] / [E_local, hidden, inter] passed through
    ``transform_weights_for_mega_moe``; shared experts likewise as 2-D tensors [2 * SI, hidden] / [hidden, SI] with
    SI = intermediate_hidden * num_shared_experts of the buffer."""
    if activation != 'swiglu':
        raise RuntimeError(f'Only `swiglu` activation is supported, got `{activation}`')
    if (shared_l1_weights is None) != (shared_l2_weights is None):
        raise RuntimeError('shared_l1_weights and shared_l2_weights must be given together')
    b = sym_buffer
    shared_inter = 0
    if shared_l1_weights is not None:
        shared_inter = b.intermediate_hidden * b.num_shared_experts
        for w, shape, name in ((shared_l1_weights, (2 * shared_inter, b.hidden), 'shared_l1_weights'),
                               (shared_l2_weights, (b.hidden, shared_inter), 'shared_l2_weights')):
            if shared_inter == 0 or not (w.is_cuda and w.dtype == torch.bfloat16 and w.is_contiguous() and tuple(w.shape) == shape):
                raise RuntimeError(f'{name} must be a contiguous CUDA bfloat16 tensor of shape {shape} '
                                   '(the buffer must have been created with num_shared_experts > 0)')
    if b.mma_type != 'bf16xbf16':
        raise RuntimeError(f'the buffer was created for `{b.mma_type}`')
    num_local = b.num_experts // b.num_ranks
    for w, shape, name in ((l1_weights, (num_local, 2 * b.intermediate_hidden, b.hidden), 'l1_weights'),
                           (l2_weights, (num_local, b.hidden, b.intermediate_hidden), 'l2_weights')):
        if not (w.is_cuda and w.dtype == torch.bfloat16 and w.is_contiguous() and tuple(w.shape) == shape):
            raise RuntimeError(f'{name} must be a contiguous CUDA bfloat16 tensor of shape {shape}')
    if not (y.is_cuda and y.dtype == torch.bfloat16 and y.dim() == 2 and y.size(1) == b.hidden and y.is_contiguous()):
        raise RuntimeError('y must be a contiguous CUDA bfloat16 [num_tokens, hidden] tensor')
    stats = cumulative_local_expert_recv_stats
    if stats is not None and not (stats.dtype == torch.int32 and stats.numel() == num_local and stats.is_contiguous()):
        raise RuntimeError('cumulative_local_expert_recv_stats must be a contiguous int32 [num_local_experts] tensor')
    ptrs = (ctypes.c_uint64 * len(b.handle.buffer_ptrs))(*[int(p) for p in b.handle.buffer_ptrs])
    p = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    with torch.cuda.device(y.device):
        _lib.check(_lib.lib().dgb200_bf16_mega_moe(
            p(y), p(l1_weights), p(l2_weights), p(shared_l1_weights), p(shared_l2_weights), shared_inter, p(stats), p(b.buffer),
            ctypes.cast(ptrs, ctypes.c_void_p), b.rank,
            b.num_ranks, y.size(0), b.num_max_tokens_per_rank, b.num_experts, b.num_topk, b.hidden,
            b.intermediate_hidden, float(activation_clamp) if activation_clamp is not None else 0.0, int(fast_math),
            _lib.current_stream_ptr()))


def route_sigmoid_topk(logits: torch.Tensor, num_topk: int, topk_idx: Optional[torch.Tensor] = None,
                       topk_weights: Optional[torch.Tensor] = None):
    """Router of the benchmark layer (no reference counterpart; the reference's tests call torch.topk):
    top-k of the logits, weights = renormalised sigmoid scores. Writes into the given views (e.g. the buffer's)."""
    if not (logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()):
        raise RuntimeError('logits must be a contiguous CUDA float32 [tokens, experts] tensor')
    t, e = logits.shape
    if topk_idx is None:
        topk_idx = torch.empty((t, num_topk), dtype=torch.int64, device=logits.device)
    if topk_weights is None:
        topk_weights = torch.empty((t, num_topk), dtype=torch.float32, device=logits.device)
    assert topk_idx.is_contiguous() and topk_weights.is_contiguous()
    with torch.cuda.device(logits.device):
        _lib.check(_lib.lib().dgb200_route_sigmoid_topk(
            ctypes.c_void_p(logits.data_ptr()), t, e, num_topk, ctypes.c_void_p(topk_idx.data_ptr()),
            ctypes.c_void_p(topk_weights.data_ptr()), _lib.current_stream_ptr()))
    return topk_idx, topk_weights
