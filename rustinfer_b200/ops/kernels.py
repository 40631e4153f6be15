"""Typed Python fronts of the CUDA kernels.  Each checks what the kernel assumes
(device, dtype, layout, sizes) and raises instead of computing something wrong."""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import library as L
from .library import KernelError, check, dtype_code, require_cuda, stream_ptr


def _p(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _i32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[t,:] (fp32) = table[ids[t],:]."""
    require_cuda(ids, table, out)
    _i32(ids, "ids"); _contig(table, "table"); _contig(out, "out")
    if out.dtype != torch.float32 or out.shape != (ids.numel(), table.shape[1]):
        raise KernelError(f"embed_gather: out must be fp32 [{ids.numel()}, {table.shape[1]}]")
    check(L.core().ri_embed_gather(_p(ids), _p(table), dtype_code(table.dtype), _p(out),
                                   ids.numel(), table.shape[1], table.shape[0], stream_ptr()),
          "embed_gather")


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """h (fp32 [T,d]) += delta; out = rmsnorm(h) * weight in out's dtype.  With `rows`
    (int32 [R]) only those rows are normed into out [R,d] and h is left as it is."""
    require_cuda(h, delta, weight, out, rows)
    d = h.shape[-1]
    _contig(h, "h"); _contig(out, "out"); _contig(weight, "weight"); _i32(rows, "rows")
    if h.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the residual stream is fp32")
    if weight.numel() != d:
        raise KernelError(f"add_rmsnorm: weight has {weight.numel()} elements, rows have {d}")
    n_rows = h.shape[0] if rows is None else rows.numel()
    if out.shape != (n_rows, d):
        raise KernelError(f"add_rmsnorm: out must be [{n_rows}, {d}], got {tuple(out.shape)}")
    if delta is not None:
        _contig(delta, "delta")
        if delta.shape != h.shape or delta.dtype != out.dtype:
            raise KernelError("add_rmsnorm: delta must match h's shape and out's dtype")
    check(L.core().ri_add_rmsnorm(_p(h), _p(delta), _p(weight), dtype_code(weight.dtype), float(eps),
                                  _p(out), dtype_code(out.dtype), _p(rows), n_rows, d, stream_ptr()),
          "add_rmsnorm")


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> None:
    require_cuda(h, delta)
    _contig(h, "h"); _contig(delta, "delta")
    if h.dtype != torch.float32 or h.shape != delta.shape:
        raise KernelError("residual_add: h is fp32 and delta has its shape")
    check(L.core().ri_residual_add(_p(h), _p(delta), dtype_code(delta.dtype), h.numel(), stream_ptr()),
          "residual_add")


def rope_scatter(qkv: torch.Tensor, positions: torch.Tensor, cos: Optional[torch.Tensor],
                 sin: Optional[torch.Tensor], slot_of_token: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                 num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int) -> None:
    """Rotate q (in place) and k of qkv [T, (Hq+2Hkv)*hd]; write k,v of token t into the
    cache [pages, 2, Hkv, page, hd] at slot_of_token[t] (page*page_size + offset; <0 skips).
    With rotary_dim 0 (cos and sin None) nothing is rotated: k and v are only written."""
    require_cuda(qkv, positions, cos, sin, slot_of_token, cache)
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token")
    T = qkv.shape[0]
    if qkv.stride(1) != 1 or qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError("rope_scatter: qkv must be [T, (Hq+2Hkv)*head_dim] with unit column stride")
    if rotary_dim % 2 or not 0 <= rotary_dim <= head_dim:
        raise KernelError(f"rope_scatter: rotary_dim {rotary_dim} must be even and at most head_dim")
    if rotary_dim and (cos is None or sin is None or cos.dtype != torch.float32 or sin.dtype != torch.float32
                       or cos.shape[1] != rotary_dim // 2):
        raise KernelError("rope_scatter: cos/sin are fp32 [positions, rotary_dim/2]")
    page = 0
    if cache is not None:
        _contig(cache, "cache")
        if cache.dtype != qkv.dtype or cache.dim() != 5 or cache.shape[1] != 2 or \
                cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
            raise KernelError("rope_scatter: cache must be [pages, 2, Hkv, page, head_dim] of qkv's dtype")
        page = cache.shape[3]
    check(L.core().ri_rope_scatter(_p(qkv), dtype_code(qkv.dtype), qkv.stride(0), _p(positions),
                                   _p(cos), _p(sin), _p(slot_of_token), _p(cache), T, num_heads,
                                   num_kv_heads if cache is not None else 0, head_dim, rotary_dim,
                                   max(page, 1), stream_ptr()), "rope_scatter")


def silu_mul(gu: torch.Tensor, out: torch.Tensor) -> None:
    require_cuda(gu, out)
    _contig(gu, "gu"); _contig(out, "out")
    T, two_i = gu.shape
    if two_i % 2 or out.shape != (T, two_i // 2) or out.dtype != gu.dtype:
        raise KernelError("silu_mul: gu is [T, 2I], out [T, I] of the same dtype")
    check(L.core().ri_silu_mul(_p(gu), _p(out), dtype_code(gu.dtype), T, two_i // 2, stream_ptr()),
          "silu_mul")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T, exact fp32."""
    require_cuda(a, w, out)
    for t, n in ((a, "a"), (w, "w"), (out, "out")):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_f32: {n} must be a 2-d fp32 tensor with unit column stride")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    check(L.core().ri_gemm_f32(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0),
                               M, N, K, stream_ptr()), "gemm_f32")


# ------------------------------------------------------------ tcgen05 bf16 matrix product
EPI_BF16, EPI_F32, EPI_SILU, EPI_RESIDUAL = 0, 1, 2, 3
EPI_RELU2 = 5             # max(x, 0)^2 of the fp32 sums, stored bf16
_tc_state = {}
_TC_WORKSPACE_FLOATS = 8 << 20
_TC_COUNTERS = 1 << 14


def gemm_tc_state(device: torch.device):
    """(workspace fp32, tile counters int32, error flag int32, meeting buffer fp32) of the
    tensor-core GEMM on a device; made once, so that captured graphs keep valid addresses.
    The meeting buffer (two 256 x 256 fp32 tiles per pair of SMs) is where CTA pairs that
    share a tile's sum over K leave their parts."""
    st = _tc_state.get(device)
    if st is None:
        st = (torch.empty(_TC_WORKSPACE_FLOATS, dtype=torch.float32, device=device),
              torch.zeros(_TC_COUNTERS, dtype=torch.int32, device=device),
              torch.zeros(1, dtype=torch.int32, device=device),
              torch.zeros(L.num_sms() * 65536, dtype=torch.float32, device=device))
        _tc_state[device] = st
    return st


def gemm_tc_error(device: torch.device) -> int:
    """The code a timed-out wait inside the tensor-core GEMM left (0: none); clears it."""
    st = _tc_state.get(device)
    if st is None:
        return 0
    code = int(st[2].item())
    if code:
        st[2].zero_()
        st[1].zero_()
    return code


def gemm_tc_plan(M: int, N: int, K: int, num_sms: Optional[int] = None, epilogue: int = EPI_BF16):
    """(swap, bn, splits, a_box): which operand sits on the 128-row side of the MMA, the
    tile of the other one, how many K slices, and how many rows of the 128 a tile really
    covers, so that about one even wave of CTAs covers the GPU."""
    num_sms = num_sms or L.num_sms()
    if M <= 64:
        swap, bn = 1, (16 if M <= 16 else 32 if M <= 32 else 64)
        tiles = -(-N // 128)
    else:
        swap, bn = 0, (256 if N >= 256 else 128 if N > 64 else 64 if N > 32 else 32 if N > 16 else 16)
        tiles = -(-M // 128) * -(-N // bn)
    kblocks = -(-K // 64)
    splits, a_box = 1, 128
    if tiles * 2 <= num_sms:
        splits = max(1, min(num_sms // tiles, kblocks // 4, 32))
        if epilogue != EPI_RESIDUAL:                       # slices meet in the workspace
            while splits > 1 and tiles * splits * bn * 128 > _TC_WORKSPACE_FLOATS:
                splits -= 1
    elif swap:
        # few tokens, no K slices: shrink the tiles until the last wave is as full as the others
        waves = -(-tiles // num_sms)
        a_box = min(128, max(64, 8 * -(-N // (8 * waves * num_sms))))
    return swap, bn, splits, a_box


def gemm_tc_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.is_contiguous() and w.is_contiguous() and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_BF16,
            plan=None, num_sms: Optional[int] = None) -> None:
    """out = x[M,K] @ w[N,K]^T on the tcgen05 tensor cores, bf16 inputs, fp32 accumulation.
    epilogue: EPI_BF16 / EPI_F32 store into out [M,N]; EPI_SILU stores silu(gate)*up into
    out [M,N/2] for a weight whose rows alternate gate_j, up_j; EPI_RESIDUAL adds into the
    fp32 out [M,N]; EPI_RELU2 stores max(x, 0)^2 as bf16."""
    require_cuda(x, w, out)
    if not gemm_tc_supports(x, w):
        raise KernelError("gemm_tc: contiguous, 16-byte aligned bfloat16 x [M,K] and w [N,K] with K a multiple of 8")
    M, Kd = x.shape
    N = w.shape[0]
    if w.shape[1] != Kd or out.stride(1) != 1:
        raise KernelError(f"gemm_tc: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    cols = N // 2 if epilogue == EPI_SILU else N
    want = torch.bfloat16 if epilogue in (EPI_BF16, EPI_SILU, EPI_RELU2) else torch.float32
    if out.dtype != want or out.shape != (M, cols) or (epilogue == EPI_SILU and N % 2):
        raise KernelError(f"gemm_tc: out must be {want} [{M}, {cols}] for epilogue {epilogue}")
    plan = plan or gemm_tc_plan(M, N, Kd, num_sms, epilogue)
    swap, bn, splits = plan[:3]
    a_box = plan[3] if len(plan) > 3 else 128
    ws, counters, err, meeting = gemm_tc_state(x.device)
    tiles = (-(-N // a_box)) * (-(-M // bn)) if swap else (-(-M // a_box)) * (-(-N // bn))
    meets = splits > 1 and epilogue != EPI_RESIDUAL
    if tiles > counters.numel() or (meets and tiles * splits * bn * 128 > ws.numel()):
        raise KernelError("gemm_tc: the split-K workspace is too small for this plan")
    check(L.gemm_tc().ri_gemm_tc(_p(x), _p(w), M, N, Kd, _p(out), out.stride(0), epilogue, swap, bn, splits,
                                 a_box, _p(ws), _p(counters), _p(err), _p(meeting), stream_ptr()), "gemm_tc")


def gemm_tc_rope(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                 cos: torch.Tensor, sin: torch.Tensor, slot_of_token: Optional[torch.Tensor],
                 cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """q, k, v = x[M,K] @ w[N,K]^T with the rotary encoding and the write of keys and values into
    their pages in the product's epilogue: q_out [M, num_heads * head_dim] bf16 gets the rotated
    queries.  `num_kv_heads` 0 (no slots, no cache) for a layer that keeps no keys.  False when the
    kernel does not take the product (fewer than 512 tokens, another head size): nothing was
    launched, and the caller runs the product and `rope_scatter` one after the other."""
    require_cuda(x, w, q_out, positions, cos, sin)
    M, Kd = x.shape
    N = w.shape[0]
    if (M < 512 or head_dim not in (64, 128) or not gemm_tc_supports(x, w) or cos.dtype != torch.float32
            or cos.shape[-1] * 2 != head_dim or q_out.dtype != torch.bfloat16 or q_out.stride(1) != 1
            or N != (num_heads + 2 * num_kv_heads) * head_dim or N < 256):
        return False
    page = 0
    if num_kv_heads > 0:
        if slot_of_token is None or cache is None:
            raise KernelError("gemm_tc_rope: a layer with keys needs the tokens' slots and the cache")
        require_cuda(slot_of_token, cache)
        page = cache.shape[3]
    _ws, counters, err, _meet = gemm_tc_state(x.device)
    st = L.gemm_tc().ri_gemm_tc_rope(_p(x), _p(w), M, N, Kd, _p(q_out), q_out.stride(0), _p(positions), _p(cos), _p(sin),
                                     _p(slot_of_token) if num_kv_heads > 0 else None,
                                     _p(cache) if num_kv_heads > 0 else None, num_heads, num_kv_heads, head_dim,
                                     page, _p(counters), _p(err), stream_ptr())
    if st == 801:                                           # not supported for this product: nothing was launched
        return False
    check(st, "gemm_tc_rope")
    return True


class _ChainPhase(ctypes.Structure):
    _fields_ = [("w", ctypes.c_void_p), ("N", ctypes.c_int), ("K", ctypes.c_int), ("x_kind", ctypes.c_int),
                ("ld_x", ctypes.c_int), ("x_rows", ctypes.c_int), ("x", ctypes.c_void_p), ("norm_w", ctypes.c_void_p),
                ("norm_w_dtype", ctypes.c_int), ("eps", ctypes.c_float), ("out_kind", ctypes.c_int),
                ("ld_out", ctypes.c_int), ("out", ctypes.c_void_p), ("xn", ctypes.c_void_p),
                ("rowsq", ctypes.c_void_p), ("part_lse", ctypes.c_void_p), ("part_splits", ctypes.c_int),
                ("part_heads", ctypes.c_int), ("part_head_dim", ctypes.c_int)]


class _ChainRope(ctypes.Structure):
    _fields_ = [("qkv", ctypes.c_void_p), ("ld", ctypes.c_int), ("positions", ctypes.c_void_p),
                ("cos_t", ctypes.c_void_p), ("sin_t", ctypes.c_void_p), ("slot_of_token", ctypes.c_void_p),
                ("q_out", ctypes.c_void_p), ("ld_q", ctypes.c_int), ("cache", ctypes.c_void_p),
                ("Hq", ctypes.c_int), ("Hkv", ctypes.c_int), ("hd", ctypes.c_int), ("rot", ctypes.c_int),
                ("page_size", ctypes.c_int)]


CHAIN_ADD_F32, CHAIN_SILU_BF16, CHAIN_BF16 = 0, 1, 2
CHAIN_MAX_TOKENS, CHAIN_MAX_PRODUCTS = 64, 6


class ChainProduct:
    """One product of a `decode_chain`: out (+)= f(x) w^T.  `x` is a bf16 matrix [M, K], or,
    with `norm=(weight, eps)`, the fp32 stream [M, K] whose RMS norm times `weight` is the
    operand.  `out_kind`: CHAIN_ADD_F32 adds into an fp32 matrix; CHAIN_SILU_BF16 stores
    silu(gate) * up of a weight whose rows alternate gate_j, up_j into bf16 [M, N/2];
    CHAIN_BF16 stores bf16 [M, N]."""

    def __init__(self, w: torch.Tensor, x: torch.Tensor, out: torch.Tensor, out_kind: int, norm=None,
                 x_rows: Optional[int] = None, xn: Optional[torch.Tensor] = None,
                 rowsq: Optional[torch.Tensor] = None, partials=None):
        self.w, self.x, self.out, self.out_kind, self.norm = w, x, out, out_kind, norm
        # partials = (part_o, part_lse, splits, heads, head_dim): instead of reading `x`, the product
        # merges the key ranges a split decode attention left (steps of up to 16 tokens, one token an entry)
        self.partials = partials
        if partials is not None:
            po, pl, splits, heads, hd = partials
            M = x.shape[0]
            if (norm is not None or po.dtype != torch.float32 or pl.dtype != torch.float32 or heads * hd != w.shape[1]
                    or hd % 8 or po.numel() < M * heads * splits * hd or pl.numel() < M * heads * splits
                    or po.data_ptr() % 16 or M > 16):
                raise KernelError("decode_chain: the partial attention results do not fit this product")
        # steps of more than 16 tokens with a norm: room for the normed operand, bf16 [64, K], and
        # for the rows' sums of squares, fp32 [64], zero before the first use (the kernel leaves it zero)
        self.xn, self.rowsq = xn, rowsq
        if norm is not None and xn is not None and (xn.dtype != torch.bfloat16 or tuple(xn.shape) != (CHAIN_MAX_TOKENS, w.shape[1])
                                                  or not xn.is_contiguous() or rowsq is None or rowsq.dtype != torch.float32
                                                  or rowsq.numel() != CHAIN_MAX_TOKENS):
            raise KernelError("decode_chain: the room for the normed operand does not fit")
        # rows behind x that may be read (not used): a bf16 x is fetched in boxes of 8, 16 or 32 rows
        self.x_rows = x.shape[0] if x_rows is None else x_rows
        N, Kd = w.shape
        want_x = torch.float32 if norm is not None else torch.bfloat16
        cols = N // 2 if out_kind == CHAIN_SILU_BF16 else N
        want_o = torch.float32 if out_kind == CHAIN_ADD_F32 else torch.bfloat16
        if (w.dtype != torch.bfloat16 or not w.is_contiguous() or x.dtype != want_x or x.shape[1] != Kd
                or x.stride(1) != 1 or out.dtype != want_o or out.shape[1] != cols or out.stride(1) != 1
                or x.shape[0] != out.shape[0] or (norm is not None and norm[0].numel() != Kd)):
            raise KernelError(f"decode_chain: product w{tuple(w.shape)} x{tuple(x.shape)} {x.dtype} "
                              f"out{tuple(out.shape)} {out.dtype} does not fit together")

    def fill(self, c: "_ChainPhase") -> None:
        c.w, c.N, c.K = self.w.data_ptr(), self.w.shape[0], self.w.shape[1]
        c.x, c.ld_x, c.x_kind = self.x.data_ptr(), self.x.stride(0), 1 if self.norm is not None else 0
        c.x_rows = self.x_rows
        if self.norm is not None:
            c.norm_w, c.norm_w_dtype, c.eps = self.norm[0].data_ptr(), dtype_code(self.norm[0].dtype), float(self.norm[1])
        else:
            c.norm_w, c.norm_w_dtype, c.eps = None, 0, 0.0
        c.out, c.ld_out, c.out_kind = self.out.data_ptr(), self.out.stride(0), self.out_kind
        c.xn = self.xn.data_ptr() if self.xn is not None else None
        c.rowsq = self.rowsq.data_ptr() if self.rowsq is not None else None
        if self.partials is not None:
            po, pl, splits, heads, hd = self.partials
            c.x_kind, c.x, c.part_lse = 2, po.data_ptr(), pl.data_ptr()
            c.part_splits, c.part_heads, c.part_head_dim = int(splits), int(heads), int(hd)
        else:
            c.part_lse, c.part_splits, c.part_heads, c.part_head_dim = None, 0, 0, 0


class ChainRope:
    """The tail of a chain whose last product added q, k, v rows into the fp32 matrix `qkv`
    [M, (Hq + 2 Hkv) * hd]: rotate q and k, write q (bf16) into `q_out`, k and v into the pages
    of `cache` at `slot_of_token` (-1: not written), and put `qkv` back to zero."""

    def __init__(self, qkv, positions, cos_t, sin_t, slot_of_token, q_out, cache, Hq, Hkv, hd, rot):
        self.__dict__.update(locals())
        if qkv.dtype != torch.float32 or q_out.dtype != torch.bfloat16 or qkv.shape[1] != (Hq + 2 * Hkv) * hd \
                or q_out.shape[1] != Hq * hd or (cache is not None and (cache.dtype != torch.bfloat16 or cache.dim() != 5
                                                                      or cache.shape[2] != Hkv or cache.shape[4] != hd)):
            raise KernelError("decode_chain: the rotary tail's buffers do not fit together")

    def fill(self, c: "_ChainRope") -> None:
        c.qkv, c.ld = self.qkv.data_ptr(), self.qkv.stride(0)
        c.positions, c.cos_t, c.sin_t = self.positions.data_ptr(), self.cos_t.data_ptr(), self.sin_t.data_ptr()
        c.slot_of_token = self.slot_of_token.data_ptr() if self.slot_of_token is not None else None
        c.q_out, c.ld_q = self.q_out.data_ptr(), self.q_out.stride(0)
        c.cache = self.cache.data_ptr() if self.cache is not None else None
        c.Hq, c.Hkv, c.hd, c.rot = self.Hq, self.Hkv, self.hd, self.rot
        c.page_size = self.cache.shape[3] if self.cache is not None else 1


_chain_state: Dict[torch.device, torch.Tensor] = {}


def _chain_barrier(device: torch.device) -> torch.Tensor:
    bar = _chain_state.get(device)
    if bar is None:
        bar = torch.zeros(2, dtype=torch.int32, device=device)
        _chain_state[device] = bar
    return bar


def _chain_array(products: Sequence[ChainProduct]):
    arr = (_ChainPhase * len(products))()
    for c, pr in zip(arr, products):
        pr.fill(c)
    return arr


def decode_chain_fits(products: Sequence[ChainProduct], tokens: int, num_sms: int) -> bool:
    """Whether `decode_chain` can run these products for this many tokens."""
    if not 1 <= len(products) <= CHAIN_MAX_PRODUCTS or not 1 <= tokens <= CHAIN_MAX_TOKENS:
        return False
    lib = L.gemm_tc()
    lib.ri_decode_chain_fits.restype = ctypes.c_int
    return lib.ri_decode_chain_fits(ctypes.cast(_chain_array(products), ctypes.c_void_p), len(products),
                                    tokens, num_sms) > 0


def decode_chain(products: Sequence[ChainProduct], rope: Optional[ChainRope], tokens: int, num_sms: int) -> None:
    """Run the products one after the other for the first `tokens` rows of their matrices in
    one cooperative kernel (see csrc/decode_chain.cu), then the rotary tail if given."""
    dev = products[0].w.device
    arr = _chain_array(products)
    rp = None
    if rope is not None:
        rs = _ChainRope()
        rope.fill(rs)
        rp = ctypes.cast(ctypes.pointer(rs), ctypes.c_void_p)
    err = gemm_tc_state(dev)[2]
    check(L.gemm_tc().ri_decode_chain(ctypes.cast(arr, ctypes.c_void_p), len(products), rp, tokens,
                                      _p(_chain_barrier(dev)), _p(err), num_sms, stream_ptr()), "decode_chain")


def attention_plain(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                    cu_q: torch.Tensor, kv_len: torch.Tensor, tile_entry: torch.Tensor,
                    tile_q0: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                    scale: float, window: Optional[int], block: Optional[int] = None,
                    value_dim: Optional[int] = None, sink: bool = False, softcap: Optional[float] = None,
                    sink_values: Optional[torch.Tensor] = None, maps: int = 1, value_in_key: bool = False,
                    slopes: Optional[torch.Tensor] = None) -> None:
    """q [T, >=Hq*hd] (may be a column view of the qkv buffer), out [T, Hq*vd].  `block`: a query
    sees only the keys of its own block of that many positions (counted from 0).  `value_dim`:
    size of a value where it is not the keys'; the cache is then [pages, Hkv*page*(hd+vd)].  `sink`:
    the softmax's denominator has one added (a key of score 0 without a value); with `sink_values`
    (fp32 [Hq]) it has exp(sink_values[h]) added instead.  `softcap` c: score <- c tanh(score / c).
    `maps` m: every head has m attention maps with queries and keys of their own over one set of
    values; `num_heads` counts query heads with their maps ([head][map]), `num_kv_heads` the value
    heads, and the cache holds Hkv*m key heads ([kv head][map]).  `value_in_key`: a key's value is
    its own first `value_dim` channels, and the cache holds keys only.  `slopes` (fp32 [Hq]): a linear
    distance bias, slopes[h] * (query position - key position) taken off head h's scores after scale
    and cap.  `out` may be fp32 whatever the cache's dtype."""
    require_cuda(q, out, cache, block_table, cu_q, kv_len, tile_entry, tile_q0, sink_values, slopes)
    _slopes_ok(slopes, num_heads)
    for t, n in ((block_table, "block_table"), (cu_q, "cu_q"), (kv_len, "kv_len"),
                 (tile_entry, "tile_entry"), (tile_q0, "tile_q0")):
        _i32(t, n)
    vd = value_dim or head_dim
    page_size = _attention_common(q, out, cache, num_heads, num_kv_heads, head_dim, vd, sink_values, maps, value_in_key)
    lib = L.attention_plain(head_dim, vd)
    check(lib.ri_attention_plain_ex(_p(q), q.stride(0), _p(out), out.stride(0), _p(cache),
                                    dtype_code(cache.dtype), _p(block_table), block_table.stride(0),
                                    _p(cu_q), _p(kv_len), _p(tile_entry), _p(tile_q0), tile_entry.numel(),
                                    num_heads, num_kv_heads, page_size, float(scale),
                                    int(window) if window else 0, int(block) if block else 0, 1 if sink else 0,
                                    float(softcap) if softcap else 0.0, _p(sink_values), int(maps),
                                    1 if value_in_key else 0, 1 if out.dtype == torch.float32 else 0, _p(slopes),
                                    stream_ptr()),
          "attention_plain")


def _slopes_ok(slopes: Optional[torch.Tensor], num_heads: int) -> None:
    if slopes is not None and (slopes.dtype != torch.float32 or slopes.numel() != num_heads or not slopes.is_contiguous()):
        raise KernelError("attention: slopes is fp32 [heads]")


def _attention_common(q, out, cache, num_heads, num_kv_heads, head_dim, vd, sink_values, maps, value_in_key) -> int:
    """Checks the fp32-arithmetic attention kernels share; returns the cache's page size."""
    if q.stride(1) != 1 or out.stride(1) != 1 or q.dtype != cache.dtype or out.dtype not in (cache.dtype, torch.float32):
        raise KernelError("attention: q and cache share a dtype, out has it or is fp32; q and out have unit column stride")
    _contig(cache, "cache")
    if maps < 1 or num_heads % (num_kv_heads * maps):
        raise KernelError("attention: heads (with their maps) must be a multiple of kv heads times maps")
    if value_in_key and (maps != 1 or vd > head_dim):
        raise KernelError("attention: values inside the keys are the keys' first channels, one map a head")
    if sink_values is not None and (sink_values.dtype != torch.float32 or sink_values.numel() != num_heads
                                    or not sink_values.is_contiguous()):
        raise KernelError("attention: sink_values is fp32 [heads]")
    return paged_cache_page_size(cache, num_kv_heads, head_dim, vd, maps, value_in_key)


def attention_single_supports(num_heads: int, num_kv_heads: int, head_dim: int, value_dim: Optional[int] = None,
                              maps: int = 1) -> bool:
    """Whether the single-token attention kernel takes this geometry (up to 16 query heads a key head,
    values up to 128 wide)."""
    return bool(L.attention_plain(head_dim, value_dim or head_dim).ri_attention_single_supports(num_heads, num_kv_heads * maps))


def attention_single(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                     cu_q: torch.Tensor, kv_len: torch.Tensor, entry_list: torch.Tensor, num_heads: int,
                     num_kv_heads: int, head_dim: int, scale: float, window: Optional[int],
                     block: Optional[int] = None, value_dim: Optional[int] = None, sink: bool = False,
                     splits: int = 1, part: Optional[torch.Tensor] = None, softcap: Optional[float] = None,
                     sink_values: Optional[torch.Tensor] = None, maps: int = 1, value_in_key: bool = False,
                     slopes: Optional[torch.Tensor] = None) -> None:
    """Attention of the entries that bring one token (`entry_list`, int32; -1 skips): fp32 arithmetic, a kv
    head's keys and values read once for all its query heads.  Arguments as `attention_plain`.  `splits` > 1
    cuts every entry's keys into that many ranges, a CTA each, joined by a second launch through `part`
    (fp32, `attention_single_scratch_floats` long)."""
    require_cuda(q, out, cache, block_table, cu_q, kv_len, entry_list, part, sink_values, slopes)
    _slopes_ok(slopes, num_heads)
    if splits > 1 and (part is None or part.dtype != torch.float32 or not part.is_contiguous() or
                       part.numel() < attention_single_scratch_floats(entry_list.numel(), num_heads, value_dim or head_dim, splits)):
        raise KernelError("attention_single: the scratch for the key ranges is too small")
    for t, n in ((block_table, "block_table"), (cu_q, "cu_q"), (kv_len, "kv_len"), (entry_list, "entry_list")):
        _i32(t, n)
    vd = value_dim or head_dim
    page_size = _attention_common(q, out, cache, num_heads, num_kv_heads, head_dim, vd, sink_values, maps, value_in_key)
    lib = L.attention_plain(head_dim, vd)
    check(lib.ri_attention_single_ex(_p(q), q.stride(0), _p(out), out.stride(0), _p(cache), dtype_code(cache.dtype),
                                     _p(block_table), block_table.stride(0), _p(cu_q), _p(kv_len), _p(entry_list),
                                     entry_list.numel(), num_heads, num_kv_heads, page_size, float(scale),
                                     int(window) if window else 0, int(block) if block else 0, 1 if sink else 0,
                                     int(splits), _p(part) if splits > 1 else None,
                                     float(softcap) if softcap else 0.0, _p(sink_values), int(maps),
                                     1 if value_in_key else 0, 1 if out.dtype == torch.float32 else 0, _p(slopes),
                                     stream_ptr()),
          "attention_single", 2 if splits > 1 else 1)


def attention_rows_supports(head_dim: int, value_dim: int, value_in_key: bool = False) -> bool:
    """Whether `attention_rows` takes keys of `head_dim` and values of `value_dim` (multiples of 16, keys up to 576,
    values up to 256; values inside the keys are no wider than the keys)."""
    return L.attention_rows_supports(head_dim, value_dim, value_in_key)


def attention_rows_tokens_per_tile(num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, maps: int = 1) -> int:
    """Tokens of one tile of `attention_rows`: 64 rows over the query heads that share a key head."""
    n = int(L.attention_rows(head_dim, value_dim).ri_attention_rows_tokens_per_tile(num_heads, num_kv_heads, maps))
    if n <= 0:
        raise KernelError("attention_rows: heads (with their maps) must be a multiple of kv heads times maps")
    return n


def attention_rows(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                   cu_q: torch.Tensor, kv_len: torch.Tensor, tile_entry: torch.Tensor, tile_tok0: torch.Tensor,
                   num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: Optional[int],
                   value_dim: Optional[int] = None, sink: bool = False, softcap: Optional[float] = None,
                   sink_values: Optional[torch.Tensor] = None, maps: int = 1, value_in_key: bool = False,
                   splits: int = 1, part: Optional[torch.Tensor] = None, slopes: Optional[torch.Tensor] = None) -> None:
    """`attention_plain` on the tensor cores for a bf16 cache: the scores are fp32 sums of products of bf16 q and
    k, cap, mask and softmax are fp32, and the softmax weights meet the bf16 values unrounded (three bf16 pieces a
    weight).  Arguments as there, without `block`; tiles hold `attention_rows_tokens_per_tile` tokens.  `splits` > 1
    cuts every tile's keys into that many ranges, a CTA each, joined by a second launch through `part` (fp32,
    `attention_rows_scratch_floats` long): for few tiles over many keys."""
    require_cuda(q, out, cache, block_table, cu_q, kv_len, tile_entry, tile_tok0, sink_values, part, slopes)
    _slopes_ok(slopes, num_heads)
    for t, n in ((block_table, "block_table"), (cu_q, "cu_q"), (kv_len, "kv_len"),
                 (tile_entry, "tile_entry"), (tile_tok0, "tile_tok0")):
        _i32(t, n)
    vd = value_dim or head_dim
    if cache.dtype != torch.bfloat16 or q.stride(0) % 8 or q.data_ptr() % 16 or cache.data_ptr() % 16:
        raise KernelError("attention_rows: a bf16 cache and q rows that start on 16-byte boundaries")
    if out.dtype == torch.float32 and (out.stride(0) % 2 or out.data_ptr() % 8):
        raise KernelError("attention_rows: fp32 out rows start on 8-byte boundaries")
    page_size = _attention_common(q, out, cache, num_heads, num_kv_heads, head_dim, vd, sink_values, maps, value_in_key)
    if splits > 1 and (part is None or part.dtype != torch.float32 or not part.is_contiguous() or part.data_ptr() % 16 or
                       part.numel() < attention_rows_scratch_floats(tile_entry.numel(), num_heads, num_kv_heads, vd, maps, splits)):
        raise KernelError("attention_rows: the scratch for the key ranges is too small")
    check(L.attention_rows(head_dim, vd).ri_attention_rows(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(cache), _p(block_table), block_table.stride(0), _p(cu_q),
        _p(kv_len), _p(tile_entry), _p(tile_tok0), tile_entry.numel(), num_heads, num_kv_heads, page_size, float(scale),
        int(window) if window else 0, 1 if sink else 0, float(softcap) if softcap else 0.0, _p(sink_values), int(maps),
        1 if value_in_key else 0, 1 if out.dtype == torch.float32 else 0, int(splits), _p(part) if splits > 1 else None,
        _p(slopes), stream_ptr()), "attention_rows", 2 if splits > 1 else 1)


def attention_rows_ctas_per_sm(head_dim: int, value_dim: int, value_in_key: bool, out_dtype: torch.dtype) -> int:
    """CTAs of `attention_rows` that one SM holds at once, asked of the driver (at least 1)."""
    n = L.attention_rows(head_dim, value_dim).ri_attention_rows_ctas_per_sm(1 if value_in_key else 0,
                                                                             1 if out_dtype == torch.float32 else 0)
    return max(1, int(n))


def attention_rows_scratch_floats(tiles: int, num_heads: int, num_kv_heads: int, value_dim: int, maps: int, splits: int) -> int:
    """Elements of `attention_rows`' scratch: [tiles][key heads * CTAs a key head][64 rows][splits][value_dim + 2]."""
    if splits <= 1:
        return 0
    group = num_heads // (num_kv_heads * maps)
    return tiles * num_kv_heads * maps * (-(-group // min(group, 64))) * 64 * splits * (value_dim + 2)


def attention_single_scratch_floats(entries: int, num_heads: int, value_dim: int, splits: int) -> int:
    return entries * num_heads * splits * (value_dim + 2)


def paged_cache_page_size(cache: torch.Tensor, num_kv_heads: int, head_dim: int, value_dim: int, maps: int = 1,
                          value_in_key: bool = False) -> int:
    """Tokens a page of `cache` holds: [pages, 2, Hkv, page, hd] when keys and values have one size,
    [pages, page * (Hkv*maps*hd + Hkv*vd)] (a page's keys, then its values) when they differ or a value
    head serves several key heads, [pages, page * Hkv*hd] when the values lie inside the keys."""
    if cache.dim() == 5:
        if (value_dim != head_dim or maps != 1 or value_in_key or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads
                or cache.shape[4] != head_dim):
            raise KernelError("attention: cache must be [pages, 2, Hkv, page, head_dim]")
        return cache.shape[3]
    per_token = num_kv_heads * maps * head_dim + (0 if value_in_key else num_kv_heads * value_dim)
    if cache.dim() != 2 or cache.shape[1] % per_token:
        raise KernelError("attention: cache must be [pages, page * (key heads * head_dim + value heads * value_dim)]")
    return cache.shape[1] // per_token


# ------------------------------------- depth average, short convolutions, the gated linear recurrent unit
def _f32_vec(t: Optional[torch.Tensor], n: int, name: str) -> None:
    if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
        raise KernelError(f"{name} is contiguous fp32 [{n}]")


def rms_sandwich(h_in: torch.Tensor, delta: Optional[torch.Tensor], post_w: Optional[torch.Tensor],
                 h_out: Optional[torch.Tensor], next_w: Optional[torch.Tensor], out: Optional[torch.Tensor], eps: float,
                 rows: Optional[torch.Tensor] = None, history: Optional[torch.Tensor] = None, n_prev: int = 0,
                 dwa: Optional[torch.Tensor] = None, avg_out: Optional[torch.Tensor] = None,
                 conv: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None) -> None:
    """RMS norms around a sublayer and the weighted depth average, one launch; v is a row of h_in (fp32 [T, d],
    rows may be a column view):
        delta given:  v += rms(delta) * post_w;   h_out given: h_out <- v;
        dwa given:    v <- sum_{j < n_prev} dwa[j] * history[j] + dwa[n_prev] * v;   avg_out given: avg_out <- v;
        out given:    out <- rms(v) * next_w (None: 1)
    with rms(x) = x / sqrt(mean(x^2) + eps).  Weights are fp32 (whatever a model adds to or multiplies into them is
    the caller's business); history is fp32 [layers, T, d].  `rows` (int32): only those rows are read and only
    `out` is written.  `conv` (weight fp32 [d, taps], state fp32 [slots, taps - 1, d], state_slots int32 [T]), for a
    step in which row t is the one token of entry t: out <- n + conv(n) as `short_conv` with `residual` computes it,
    the earlier inputs from state[state_slots[t]], which the new input is shifted into."""
    require_cuda(h_in, delta, post_w, h_out, next_w, out, rows, history, dwa, avg_out, *(conv or ()))
    _i32(rows, "rows")
    T, d = h_in.shape
    if h_in.dtype != torch.float32 or h_in.stride(1) != 1:
        raise KernelError("rms_sandwich: h_in is fp32 [T, d] with unit column stride")
    if delta is not None and (delta.shape != h_in.shape or delta.stride(1) != 1 or post_w is None):
        raise KernelError("rms_sandwich: delta has h_in's shape and unit column stride, and comes with post_w")
    _f32_vec(post_w, d, "rms_sandwich: post_w"); _f32_vec(next_w, d, "rms_sandwich: next_w")
    for t, n in ((h_out, "h_out"), (avg_out, "avg_out")):
        if t is not None and (t.dtype != torch.float32 or t.shape != h_in.shape or not t.is_contiguous()):
            raise KernelError(f"rms_sandwich: {n} is contiguous fp32 [T, d]")
    if dwa is not None:
        _f32_vec(dwa, n_prev + 1, "rms_sandwich: dwa")
        if n_prev and (history is None or history.dtype != torch.float32 or not history.is_contiguous()
                       or history.dim() != 3 or history.shape[0] < n_prev or tuple(history.shape[1:]) != (T, d)):
            raise KernelError("rms_sandwich: history is contiguous fp32 [>= n_prev, T, d]")
    n_rows = T if rows is None else rows.numel()
    if out is not None and (out.shape != (n_rows, d) or not out.is_contiguous()):
        raise KernelError("rms_sandwich: out is contiguous [rows, d]")
    cw = cs = cslots = None
    taps = 0
    if conv is not None:
        cw, cs, cslots = conv
        taps = cw.shape[1]
        _i32(cslots, "conv slots")
        if rows is not None or out is None or cw.dtype != torch.float32 or cw.shape[0] != d or not cw.is_contiguous() \
                or cs.dtype != torch.float32 or not cs.is_contiguous() or tuple(cs.shape[1:]) != (taps - 1, d) or cslots.numel() < T:
            raise KernelError("rms_sandwich: conv is (fp32 [d, taps], fp32 [slots, taps - 1, d], int32 [T]) and goes with out, without rows")
    check(L.core().ri_rms_sandwich(_p(h_in), h_in.stride(0), _p(delta), dtype_code(delta.dtype) if delta is not None else 0,
                                   delta.stride(0) if delta is not None else 0, _p(post_w), _p(h_out), _p(history),
                                   T * d, int(n_prev), _p(dwa), _p(avg_out), _p(next_w), _p(out),
                                   dtype_code(out.dtype) if out is not None else 0, _p(rows), n_rows, d, float(eps),
                                   _p(cw), _p(cs), _p(cslots), int(taps), stream_ptr()), "rms_sandwich")


def short_conv_max_taps() -> int:
    return int(L.core().ri_short_conv_max_taps())


def short_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
               cu_q: torch.Tensor, state_slots: torch.Tensor, out: torch.Tensor, n_entries: int, max_q_len: int,
               residual: bool, in_bias: Optional[torch.Tensor] = None) -> None:
    """A causal convolution over time on every channel, continued from a state: out[t] = (x[t] if residual) + bias +
    sum_j weight[:, j] * x[t - taps + 1 + j] over each entry's tokens (x [T, C], may be a column view; weight fp32
    [C, taps]); the taps - 1 inputs before an entry's first token come from state[slot] (fp32 [slots, taps - 1, C],
    oldest first) and the entry's last taps - 1 inputs go back there.  `in_bias` (fp32 [C]) is added to every input
    first (the state holds the sums)."""
    require_cuda(x, weight, bias, state, cu_q, state_slots, out, in_bias)
    _f32_vec(in_bias, x.shape[1], "short_conv: in_bias")
    _i32(cu_q, "cu_q"); _i32(state_slots, "state_slots")
    T, C = x.shape
    taps = weight.shape[1]
    if x.stride(1) != 1 or out.shape != x.shape or out.stride(1) != 1:
        raise KernelError("short_conv: x and out are [T, C] with unit column stride")
    if weight.dtype != torch.float32 or weight.shape[0] != C or not weight.is_contiguous():
        raise KernelError("short_conv: weight is contiguous fp32 [C, taps]")
    _f32_vec(bias, C, "short_conv: bias")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (taps - 1, C):
        raise KernelError("short_conv: state is contiguous fp32 [slots, taps - 1, C]")
    check(L.core().ri_short_conv(_p(x), dtype_code(x.dtype), x.stride(0), _p(weight), _p(bias), _p(state), _p(cu_q),
                                 _p(state_slots), _p(out), dtype_code(out.dtype), out.stride(0), int(n_entries),
                                 int(max_q_len), C, taps, 1 if residual else 0, _p(in_bias), stream_ptr()), "short_conv")


def rglru_gates(u: torch.Tensor, wa: torch.Tensor, wi: torch.Tensor, ba: torch.Tensor, bi: torch.Tensor,
                lam: torch.Tensor, decay_scale: float, a_out: torch.Tensor, x_out: torch.Tensor) -> None:
    """Gates of the real-gated linear recurrent unit: u fp32 [T, C] in `blocks` equal parts, wa / wi [blocks, bs, bs]
    ([out, in]), ba / bi / lam fp32 [C]:  r = sigmoid(wa u + ba), i = sigmoid(wi u + bi),
    a_out = exp(-decay_scale * r * softplus(lam)),  x_out = sqrt(1 - a_out^2) * i * u.  fp32 throughout."""
    require_cuda(u, wa, wi, ba, bi, lam, a_out, x_out)
    T, C = u.shape
    blocks = wa.shape[0]
    if u.dtype != torch.float32 or u.stride(1) != 1:
        raise KernelError("rglru_gates: u is fp32 [T, C] with unit column stride")
    if blocks <= 0 or C % blocks or tuple(wa.shape) != (blocks, C // blocks, C // blocks) or wi.shape != wa.shape \
            or wi.dtype != wa.dtype or not wa.is_contiguous() or not wi.is_contiguous():
        raise KernelError("rglru_gates: wa and wi are contiguous [blocks, C / blocks, C / blocks] of one dtype")
    for t, n in ((ba, "ba"), (bi, "bi"), (lam, "lam")):
        _f32_vec(t, C, "rglru_gates: " + n)
    for t in (a_out, x_out):
        if t.dtype != torch.float32 or t.shape != (T, C) or not t.is_contiguous():
            raise KernelError("rglru_gates: a_out and x_out are contiguous fp32 [T, C]")
    check(L.core().ri_rglru_gates(_p(u), u.stride(0), _p(wa), _p(wi), dtype_code(wa.dtype), _p(ba), _p(bi), _p(lam),
                                  float(decay_scale), _p(a_out), _p(x_out), T, C, blocks, stream_ptr()), "rglru_gates")


def rglru_step(u: torch.Tensor, wa: torch.Tensor, wi: torch.Tensor, ba: torch.Tensor, bi: torch.Tensor, lam: torch.Tensor,
               decay_scale: float, y: torch.Tensor, y_bias: Optional[torch.Tensor], state: torch.Tensor,
               state_slots: torch.Tensor, out: torch.Tensor, out_scale: float = 1.0) -> None:
    """`rglru_gates` and one step of `rglru_scan` in one launch, for a step in which every entry brings exactly one
    token (row t of u, y and out is entry t, its state state[state_slots[t]]).  `out_scale`: a factor on out."""
    require_cuda(u, wa, wi, ba, bi, lam, y, y_bias, state, state_slots, out)
    _i32(state_slots, "state_slots")
    T, C = u.shape
    blocks = wa.shape[0]
    if u.dtype != torch.float32 or u.stride(1) != 1 or y.dtype != torch.float32 or y.shape != (T, C) or y.stride(1) != 1:
        raise KernelError("rglru_step: u and y are fp32 [T, C] with unit column stride")
    if blocks <= 0 or C % blocks or tuple(wa.shape) != (blocks, C // blocks, C // blocks) or wi.shape != wa.shape \
            or wi.dtype != wa.dtype or not wa.is_contiguous() or not wi.is_contiguous():
        raise KernelError("rglru_step: wa and wi are contiguous [blocks, C / blocks, C / blocks] of one dtype")
    for t, n in ((ba, "ba"), (bi, "bi"), (lam, "lam"), (y_bias, "y_bias")):
        _f32_vec(t, C, "rglru_step: " + n)
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (C,) or state_slots.numel() < T:
        raise KernelError("rglru_step: state is contiguous fp32 [slots, C], one slot an entry")
    if out.shape != (T, C) or not out.is_contiguous():
        raise KernelError("rglru_step: out is contiguous [T, C]")
    check(L.core().ri_rglru_step(_p(u), u.stride(0), _p(wa), _p(wi), dtype_code(wa.dtype), _p(ba), _p(bi), _p(lam),
                                 float(decay_scale), _p(y), y.stride(0), _p(y_bias), _p(state), _p(state_slots), _p(out),
                                 dtype_code(out.dtype), T, C, blocks, float(out_scale), stream_ptr()), "rglru_step")


def rglru_scan(a: torch.Tensor, x: torch.Tensor, y: torch.Tensor, y_bias: Optional[torch.Tensor], state: torch.Tensor,
               cu_q: torch.Tensor, state_slots: torch.Tensor, out: torch.Tensor, n_entries: int,
               max_q_len: Optional[int] = None, out_scale: float = 1.0) -> None:
    """S_t = a_t * S_(t-1) + x_t per channel over each entry's tokens, from state[slot] (fp32 [slots, C]) and back
    into it; out[t] = S_t * gelu_tanh(y[t] + y_bias).  a, x fp32 [T, C] (x is scratch: it may come back holding S);
    y fp32 [T, C], may be a column view.  `max_q_len`: an upper bound of the entries' token counts (default: T);
    entries of up to 8 tokens run as one launch, longer ones as a bare walk and an element-wise launch.  `out_scale`:
    a factor on out."""
    require_cuda(a, x, y, y_bias, state, cu_q, state_slots, out)
    _i32(cu_q, "cu_q"); _i32(state_slots, "state_slots")
    T, C = a.shape
    for t in (a, x):
        if t.dtype != torch.float32 or t.shape != (T, C) or not t.is_contiguous():
            raise KernelError("rglru_scan: a and x are contiguous fp32 [T, C]")
    if y.dtype != torch.float32 or y.shape != (T, C) or y.stride(1) != 1:
        raise KernelError("rglru_scan: y is fp32 [T, C] with unit column stride")
    _f32_vec(y_bias, C, "rglru_scan: y_bias")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (C,):
        raise KernelError("rglru_scan: state is contiguous fp32 [slots, C]")
    if out.shape != (T, C) or not out.is_contiguous():
        raise KernelError("rglru_scan: out is contiguous [T, C]")
    mq = T if max_q_len is None else int(max_q_len)
    check(L.core().ri_rglru_scan(_p(a), _p(x), _p(y), y.stride(0), _p(y_bias), _p(state), _p(cu_q), _p(state_slots),
                                 _p(out), dtype_code(out.dtype), int(n_entries), C, T, mq, float(out_scale), stream_ptr()), "rglru_scan",
          1 if mq <= 8 else 2)


def sigmoid_gate(o: torch.Tensor, gate: torch.Tensor, group: int, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, j] = scale * o[t, j] * sigmoid(gate[t, j // group]): o [T, n], gate fp32 [T, n / group] (both may be column
    views).  group 1: a gate a channel; group = a head's width: a gate a head."""
    require_cuda(o, gate, out)
    T, n = o.shape
    if o.stride(1) != 1 or gate.dtype != torch.float32 or gate.stride(1) != 1 or n % group or gate.shape != (T, n // group):
        raise KernelError("sigmoid_gate: o [T, n], gate fp32 [T, n / group], unit column strides")
    if out.shape != o.shape or not out.is_contiguous():
        raise KernelError("sigmoid_gate: out is contiguous [T, n]")
    check(L.core().ri_sigmoid_gate(_p(o), dtype_code(o.dtype), o.stride(0), _p(gate), gate.stride(0), int(group), _p(out),
                                   dtype_code(out.dtype), T, n, float(scale), stream_ptr()), "sigmoid_gate")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap), fp32, in place."""
    require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("softcap: x is contiguous fp32")
    check(L.core().ri_softcap(_p(x), x.numel(), float(cap), stream_ptr()), "softcap")


def glu_pairs(pairs: torch.Tensor, out: torch.Tensor, act: Optional[Tuple[float, float]] = None) -> None:
    """pairs fp32 [rows, 2F], a row's columns alternating gate_n, up_n: out[p, n] = silu(gate) * up, or with `act`
    (limit, alpha) g' sigmoid(alpha g') (u' + 1) with g' = min(gate, limit), u' = clamp(up, -limit, limit)."""
    require_cuda(pairs, out)
    _contig(pairs, "pairs"); _contig(out, "out")
    if pairs.dtype != torch.float32 or pairs.shape[1] % 2 or out.shape != (pairs.shape[0], pairs.shape[1] // 2):
        raise KernelError("glu_pairs: pairs fp32 [rows, 2F], out [rows, F]")
    check(L.core().ri_glu_pairs(_p(pairs), _p(out), dtype_code(out.dtype), out.numel(), 1 if act else 0,
                                float(act[0]) if act else 0.0, float(act[1]) if act else 0.0, stream_ptr()), "glu_pairs")


# ------------------------------------------------ parts of decoders that are not the Llama shape
def embed_sinusoid(ids: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, freq: torch.Tensor,
                   out: torch.Tensor) -> None:
    """out[t,:] (fp32) = table[ids[t],:] + the sinusoidal vector of positions[t]; `freq` (float64,
    [ceil(d/2)]) holds the angular frequency of every (sin, cos) pair."""
    require_cuda(ids, positions, table, freq, out)
    _i32(ids, "ids"); _i32(positions, "positions"); _contig(table, "table"); _contig(out, "out")
    d = table.shape[1]
    if out.dtype != torch.float32 or out.shape != (ids.numel(), d):
        raise KernelError(f"embed_sinusoid: out must be fp32 [{ids.numel()}, {d}]")
    if freq.dtype != torch.float64 or freq.numel() != (d + 1) // 2 or positions.numel() < ids.numel():
        raise KernelError("embed_sinusoid: freq is float64 [ceil(d/2)], one position per id")
    check(L.core().ri_embed_sinusoid(_p(ids), _p(positions), _p(table), dtype_code(table.dtype), _p(freq), _p(out),
                                     ids.numel(), d, table.shape[0], stream_ptr()), "embed_sinusoid")


def sandwich_norm(h: torch.Tensor, delta: Optional[torch.Tensor], post_w: Optional[torch.Tensor],
                  post_b: Optional[torch.Tensor], next_w: Optional[torch.Tensor], next_b: Optional[torch.Tensor],
                  out: Optional[torch.Tensor], eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """Layer norm around a sublayer.  h (fp32 [T,d]) += LN(delta; post_w, post_b) when `delta` is given;
    out = LN(h; next_w, next_b) when `out` is given.  With `rows` (int32 [R]) only those rows are
    read, out is [R,d] and h is left as it is."""
    require_cuda(h, delta, post_w, post_b, next_w, next_b, out, rows)
    d = h.shape[-1]
    _contig(h, "h"); _i32(rows, "rows")
    if h.dtype != torch.float32:
        raise KernelError("sandwich_norm: the residual stream is fp32")
    n_rows = h.shape[0] if rows is None else rows.numel()
    ws = [w for w in (post_w, post_b, next_w, next_b) if w is not None]
    for w in ws:
        _contig(w, "norm weight")
        if w.numel() != d or w.dtype != ws[0].dtype:
            raise KernelError(f"sandwich_norm: norm weights have {d} elements and one dtype")
    act = None
    if delta is not None:
        _contig(delta, "delta")
        if delta.shape != h.shape:
            raise KernelError("sandwich_norm: delta has h's shape")
        act = delta.dtype
    if out is not None:
        _contig(out, "out")
        if out.shape != (n_rows, d) or (act is not None and out.dtype != act):
            raise KernelError(f"sandwich_norm: out must be [{n_rows}, {d}] of delta's dtype")
        act = out.dtype
    if act is None:
        return
    check(L.core().ri_sandwich_norm(_p(h), _p(delta), _p(post_w), _p(post_b), _p(next_w), _p(next_b), _p(out),
                                    dtype_code(act), dtype_code(ws[0].dtype) if ws else 0, _p(rows), n_rows, d,
                                    float(eps), stream_ptr()), "sandwich_norm")


def head_norm_scatter(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                      value_norm: bool, eps: float, slot_of_token: Optional[torch.Tensor],
                      cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                      value_dim: int) -> None:
    """qkv [T, Hq*hd + Hkv*hd + Hkv*vd]: q and k of every head are divided by their root mean square
    and multiplied by a weight [hd] shared by the heads (None: left as they are), v by its root
    mean square when `value_norm`; q in place, k and v into the cache at slot_of_token[t]
    (page*page_size + offset; < 0 skips)."""
    require_cuda(qkv, q_weight, k_weight, slot_of_token, cache)
    _i32(slot_of_token, "slot_of_token")
    if qkv.stride(1) != 1 or qkv.shape[1] != num_heads * head_dim + num_kv_heads * (head_dim + value_dim):
        raise KernelError("head_norm_scatter: qkv must be [T, Hq*hd + Hkv*(hd+vd)] with unit column stride")
    ws = [w for w in (q_weight, k_weight) if w is not None]
    for w in ws:
        _contig(w, "weight")
        if w.numel() != head_dim or w.dtype != ws[0].dtype:
            raise KernelError(f"head_norm_scatter: norm weights have {head_dim} elements and one dtype")
    page = 1
    if cache is not None:
        _contig(cache, "cache")
        if cache.dtype != qkv.dtype:
            raise KernelError("head_norm_scatter: cache has qkv's dtype")
        page = paged_cache_page_size(cache, num_kv_heads, head_dim, value_dim)
    check(L.core().ri_head_norm_scatter(_p(qkv), dtype_code(qkv.dtype), qkv.stride(0), _p(q_weight), _p(k_weight),
                                        dtype_code(ws[0].dtype) if ws else 0, 1 if value_norm else 0, float(eps),
                                        _p(slot_of_token), _p(cache), qkv.shape[0], num_heads, num_kv_heads,
                                        head_dim, value_dim, page, stream_ptr()), "head_norm_scatter")


def embed_rmsnorm(ids: torch.Tensor, table: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[t,:] (fp32) = table[ids[t],:] / sqrt(mean(row^2) + eps) * weight."""
    require_cuda(ids, table, weight, out)
    _i32(ids, "ids"); _contig(table, "table"); _contig(weight, "weight")
    d = table.shape[1]
    if out.dtype != torch.float32 or out.shape != (ids.numel(), d) or not out.is_contiguous() or weight.numel() != d:
        raise KernelError(f"embed_rmsnorm: out must be contiguous fp32 [{ids.numel()}, {d}], weight [{d}]")
    check(L.core().ri_embed_rmsnorm(_p(ids), _p(table), dtype_code(table.dtype), _p(weight), dtype_code(weight.dtype),
                                    float(eps), _p(out), ids.numel(), d, table.shape[0], stream_ptr()), "embed_rmsnorm")


HYPER_MAX_STREAMS = 8


def hyper_collect(streams: torch.Tensor, fresh: bool, y: Optional[torch.Tensor], mix: Optional[torch.Tensor],
                  write: Optional[torch.Tensor], read: Optional[torch.Tensor], weight: Optional[torch.Tensor],
                  eps: float, out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None) -> None:
    """Several residual streams X [S, T, d] fp32 (`fresh`: only X[0] is written yet and stands for all).
    With `y` [T, d]: X_t <- sum_s mix[s, t] X_s + write[t] y (stored unless `rows` is given).  Then
    u = sum_s read[s] X_s (`read` None: the plain sum) and out = rmsnorm(u) * weight (`weight` None: out = u).
    With `rows` (int32 [R]) only those tokens are read and out is [R, d]."""
    require_cuda(streams, y, mix, write, read, weight, out, rows)
    _contig(streams, "streams"); _i32(rows, "rows")
    if streams.dtype != torch.float32 or streams.dim() != 3:
        raise KernelError("hyper_collect: the streams are fp32 [S, T, d]")
    S, T, d = streams.shape
    if not 1 <= S <= HYPER_MAX_STREAMS:
        raise KernelError(f"hyper_collect: 1 to {HYPER_MAX_STREAMS} streams")
    if y is not None:
        _contig(y, "y")
        if y.shape != (T, d) or mix is None or write is None or tuple(mix.shape) != (S, S) or write.numel() != S \
                or mix.dtype != torch.float32 or write.dtype != torch.float32 or not mix.is_contiguous():
            raise KernelError("hyper_collect: y is [T, d], mix fp32 [S, S], write fp32 [S]")
    if read is not None and (read.numel() != S or read.dtype != torch.float32):
        raise KernelError("hyper_collect: read is fp32 [S]")
    n_rows = T if rows is None else rows.numel()
    if out is not None:
        _contig(out, "out")
        if out.shape != (n_rows, d):
            raise KernelError(f"hyper_collect: out must be [{n_rows}, {d}]")
    if weight is not None:
        _contig(weight, "weight")
        if weight.numel() != d:
            raise KernelError("hyper_collect: weight has d elements")
    check(L.core().ri_hyper_collect(_p(streams), 1 if fresh else 0, _p(y), dtype_code(y.dtype) if y is not None else 0,
                                    _p(mix), _p(write), _p(read), _p(weight),
                                    dtype_code(weight.dtype) if weight is not None else 0, float(eps), _p(out),
                                    dtype_code(out.dtype) if out is not None else 0, _p(rows), n_rows, T, d, S,
                                    stream_ptr()), "hyper_collect")


def qkv_prepare(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_weight: Optional[torch.Tensor],
                k_weight: Optional[torch.Tensor], norm_mode: int, eps: float, positions: torch.Tensor,
                cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int, interleaved: bool,
                slot_of_token: Optional[torch.Tensor], cache: Optional[torch.Tensor], q_out: torch.Tensor,
                num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, has_kv: bool,
                value_heads: Optional[int] = None) -> None:
    """qkv [T, Hq*hd (+ Hkv*hd + Hkv*vd when `has_kv`)]: add `bias` (fp32), norm q and k (`norm_mode` 0: not;
    1: every head by its own root mean square, weights [hd]; 2: all heads at once, weights [Hq*hd] and
    [Hkv*hd]), rotate the first `rotary_dim` channels of every head (pairs (2i, 2i+1) when `interleaved`, else
    (i, i + rotary_dim/2)), write q into q_out [T, Hq*hd] and k, v into the cache at slot_of_token[t].
    `value_heads`: heads of v where they are fewer than the heads of k (`num_kv_heads` then counts the key
    heads: kv heads times the attention maps of a head).  qkv may be the leading columns of wider rows."""
    require_cuda(qkv, bias, q_weight, k_weight, positions, cos, sin, slot_of_token, cache, q_out)
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token")
    T = qkv.shape[0]
    Hv = value_heads or num_kv_heads
    if num_kv_heads % Hv:
        raise KernelError("qkv_prepare: key heads are a multiple of value heads")
    cols = num_heads * head_dim + (num_kv_heads * head_dim + Hv * value_dim if has_kv else 0)
    if qkv.stride(1) != 1 or qkv.shape[1] != cols:
        raise KernelError(f"qkv_prepare: qkv must be [T, {cols}] with unit column stride")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != cols or not bias.is_contiguous()):
        raise KernelError(f"qkv_prepare: bias is fp32 [{cols}]")
    _contig(q_out, "q_out")
    if q_out.shape != (T, num_heads * head_dim):
        raise KernelError("qkv_prepare: q_out is [T, Hq*hd]")
    ws = [w for w in (q_weight, k_weight) if w is not None]
    want = {0: (0, 0), 1: (head_dim, head_dim), 2: (num_heads * head_dim, num_kv_heads * head_dim)}[norm_mode]
    for w, n in zip((q_weight, k_weight), want):
        if w is not None and (w.numel() != n or w.dtype != ws[0].dtype or not w.is_contiguous()):
            raise KernelError("qkv_prepare: the norm weights' sizes do not fit the norm mode")
    if norm_mode and (q_weight is None or (has_kv and k_weight is None)):
        raise KernelError("qkv_prepare: a norm needs its weights")
    if rotary_dim and (cos is None or sin is None or cos.dtype != torch.float32 or sin.dtype != torch.float32
                       or cos.shape[1] != rotary_dim // 2 or not cos.is_contiguous() or not sin.is_contiguous()):
        raise KernelError("qkv_prepare: cos/sin are fp32 [positions, rotary_dim/2]")
    page = 1
    if cache is not None:
        _contig(cache, "cache")
        if cache.dtype != q_out.dtype:
            raise KernelError("qkv_prepare: the cache has q_out's dtype")
        page = paged_cache_page_size(cache, Hv, head_dim, value_dim, num_kv_heads // Hv)
    check(L.core().ri_qkv_prepare(_p(qkv), dtype_code(qkv.dtype), qkv.stride(0), _p(bias), _p(q_weight), _p(k_weight),
                                  dtype_code(ws[0].dtype) if ws else 0, int(norm_mode), float(eps), _p(positions),
                                  _p(cos), _p(sin), int(rotary_dim), 1 if interleaved else 0, _p(slot_of_token), _p(cache),
                                  _p(q_out), dtype_code(q_out.dtype), T, num_heads, num_kv_heads, head_dim, value_dim,
                                  1 if has_kv else 0, page, Hv, stream_ptr()), "qkv_prepare")


# ------------------------------------------------------------------------ routed experts
def moe_route(z: Optional[torch.Tensor], correction: Optional[torch.Tensor], top: int, n_groups: int, keep: int, renorm: bool,
              ids: torch.Tensor, weights: torch.Tensor, counts: torch.Tensor, x: Optional[torch.Tensor] = None,
              router: Optional[torch.Tensor] = None, score: str = "sigmoid") -> None:
    """The `top` experts of every token (ids int32 [T, top]) and their weights (fp32 [T, top]) from router logits:
    either z [T, E] fp32 is given, or x [T, d] and the router's matrix (fp32 [E, d]) and the kernel forms z = x W^T
    itself in fp32.  Scores sigmoid(z), chosen by score + correction among the experts of the `keep` best of
    `n_groups` groups (0: no groups).  With `score` "softmax_chosen" the scores are the logits themselves and the
    weights the softmax of the chosen logits among themselves.  counts (int32 [E]) gets one added per choice."""
    if score not in ("sigmoid", "softmax_chosen"):
        raise KernelError(f"moe_route: score {score!r}")
    require_cuda(z, correction, ids, weights, counts, x, router)
    E = counts.numel()
    T = ids.shape[0]
    _contig(ids, "ids"); _contig(weights, "weights"); _i32(ids, "ids"); _i32(counts, "counts")
    if (z is None) == (x is None):
        raise KernelError("moe_route: give the logits or the router's input, not both")
    if z is not None and (z.dtype != torch.float32 or z.shape != (T, E) or not z.is_contiguous()):
        raise KernelError("moe_route: z is contiguous fp32 [T, E]")
    d = 0
    if x is not None:
        d = x.shape[1]
        if router is None or router.dtype != torch.float32 or tuple(router.shape) != (E, d) or not router.is_contiguous() \
                or not x.is_contiguous() or x.shape[0] != T:
            raise KernelError("moe_route: x is contiguous [T, d] and the router's matrix fp32 [E, d]")
    if weights.dtype != torch.float32 or ids.shape != (T, top) or weights.shape != (T, top) \
            or (correction is not None and (correction.dtype != torch.float32 or correction.numel() != E)):
        raise KernelError("moe_route: correction fp32 [E], ids int32 and weights fp32 [T, top], counts [E]")
    check(L.core().ri_moe_route(_p(z), _p(x), dtype_code(x.dtype) if x is not None else 0, _p(router), d, _p(correction), T, E,
                                int(top), int(n_groups), int(keep), 1 if renorm else 0, _p(ids), _p(weights), _p(counts),
                                1 if score == "softmax_chosen" else 0, stream_ptr()), "moe_route")


def moe_sort(ids: torch.Tensor, counts: torch.Tensor, offsets: torch.Tensor, order: torch.Tensor, place: torch.Tensor) -> None:
    """The (token, choice) pairs in expert order: offsets int32 [E + 1], order int32 [N] (pair at each place),
    place int32 [N] (place of each pair); pairs of one expert keep their order."""
    require_cuda(ids, counts, offsets, order, place)
    N, E = ids.numel(), counts.numel()
    for t, n in ((ids, "ids"), (counts, "counts"), (offsets, "offsets"), (order, "order"), (place, "place")):
        _i32(t, n); _contig(t, n)
    if offsets.numel() != E + 1 or order.numel() != N or place.numel() != N:
        raise KernelError("moe_sort: offsets [E + 1], order and place [N]")
    check(L.core().ri_moe_sort(_p(ids), _p(counts), N, E, _p(offsets), _p(order), _p(place), stream_ptr()), "moe_sort")


def moe_product(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor, order: Optional[torch.Tensor],
                top: int, gated: bool, act: Optional[Tuple[float, float]] = None) -> None:
    """Rows in expert order times their expert's matrix w [E, Ntot, K]: row p is a[order[p] // top] when `order`
    is given, else a[p].  gated: Ntot = 2N and the rows of w_e alternate gate_n, up_n: out[p][n] =
    silu(a . w_e[2n]) * (a . w_e[2n+1]); else out[p] = a w_e^T.  `act` (limit, alpha) with gated: the pair
    (g, u) becomes g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit) instead.
    fp32 sums in the order of k."""
    require_cuda(a, w, out, offsets, order)
    _contig(w, "w"); _i32(offsets, "offsets"); _i32(order, "order")
    E, Ntot, Kd = w.shape
    N = Ntot // 2 if gated else Ntot
    rows = out.shape[0]
    if a.stride(1) != 1 or a.shape[1] != Kd or out.stride(1) != 1 or out.shape[1] != N or offsets.numel() != E + 1 \
            or (order is not None and order.numel() != rows) or (order is None and a.shape[0] != rows):
        raise KernelError(f"moe_product: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    check(L.core().ri_moe_product(_p(a), dtype_code(a.dtype), a.stride(0), _p(w), dtype_code(w.dtype), _p(out),
                                  dtype_code(out.dtype), out.stride(0), _p(offsets), _p(order), int(top),
                                  1 if order is not None else 0, rows, E, N, Kd, 1 if gated else 0,
                                  1 if act else 0, float(act[0]) if act else 0.0, float(act[1]) if act else 0.0,
                                  stream_ptr()),
          "moe_product")


def moe_gather(x: torch.Tensor, order: torch.Tensor, top: int, out: torch.Tensor) -> None:
    """out[p] = x[order[p] // top]: the tokens' rows (bf16, a multiple of 8 wide) in expert order."""
    require_cuda(x, order, out)
    _contig(x, "x"); _contig(out, "out"); _i32(order, "order")
    if x.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or out.shape != (order.numel(), x.shape[1]) or x.shape[1] % 8:
        raise KernelError("moe_gather: bf16 x [T, d] and out [rows, d] with d a multiple of 8")
    check(L.core().ri_moe_gather(_p(x), _p(order), int(top), _p(out), out.shape[0], x.shape[1], stream_ptr()), "moe_gather")


def gemm_tc_grouped_supports(rows: int, n: int, k: int) -> bool:
    """Whether `gemm_tc_grouped` takes rows of k against matrices of n rows (TMA wants 16-byte row pitches)."""
    return k % 8 == 0 and n % 8 == 0


def gemm_tc_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor, epilogue: int,
                    act: Optional[Tuple[float, float]] = None) -> None:
    """Rows in groups against a matrix per group on the tcgen05 tensor cores: x [rows, K] bf16 holds the groups one
    after the other (group e: rows offsets[e] .. offsets[e+1]-1, int32 on the device), w [E, N, K] bf16.  EPI_F32 /
    EPI_BF16 store into out [rows, N]; EPI_SILU stores silu(gate) * up of matrices whose rows alternate gate_j, up_j
    into out [rows, N/2], or with `act` (limit, alpha) the clamped pair g' sigmoid(alpha g') (u' + 1)."""
    require_cuda(x, w, out, offsets)
    _contig(x, "x"); _contig(w, "w"); _contig(out, "out"); _i32(offsets, "offsets")
    E, N, Kd = w.shape
    rows = x.shape[0]
    cols = N // 2 if epilogue == EPI_SILU else N
    want = torch.float32 if epilogue == EPI_F32 else torch.bfloat16
    if (x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.shape[1] != Kd or Kd % 8 or x.data_ptr() % 16
            or w.data_ptr() % 16 or out.dtype != want or out.shape != (rows, cols) or offsets.numel() != E + 1
            or epilogue not in (EPI_BF16, EPI_F32, EPI_SILU)):
        raise KernelError(f"gemm_tc_grouped: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} {out.dtype}")
    err = gemm_tc_state(x.device)[2]
    if act is not None and epilogue != EPI_SILU:
        raise KernelError("gemm_tc_grouped: the clamped pair is a form of the gated epilogue")
    check(L.gemm_tc().ri_gemm_tc_grouped(_p(x), _p(w), rows, N, Kd, _p(out), out.stride(0), int(epilogue), _p(offsets), E,
                                         _p(err), float(act[0]) if act else 0.0, float(act[1]) if act else 0.0,
                                         stream_ptr()), "gemm_tc_grouped")


def moe_combine(Y: torch.Tensor, place: torch.Tensor, weights: torch.Tensor, shared: Optional[torch.Tensor],
                out: torch.Tensor, counts: torch.Tensor) -> None:
    """out[t] = sum_j weights[t, j] * Y[place[t * top + j]] (+ shared[t]); counts is put back to zero."""
    require_cuda(Y, place, weights, shared, out, counts)
    T, top = weights.shape
    d = Y.shape[1]
    _contig(Y, "Y"); _contig(out, "out"); _contig(weights, "weights"); _i32(place, "place"); _i32(counts, "counts")
    if Y.dtype != torch.float32 or weights.dtype != torch.float32 or Y.shape[0] != T * top or out.shape != (T, d) \
            or place.numel() != T * top or (shared is not None and (shared.shape != (T, d) or not shared.is_contiguous())):
        raise KernelError("moe_combine: Y fp32 [T*top, d], weights fp32 [T, top], shared and out [T, d]")
    check(L.core().ri_moe_combine(_p(Y), _p(place), _p(weights), _p(shared),
                                  dtype_code(shared.dtype) if shared is not None else 0, _p(out), dtype_code(out.dtype),
                                  T, top, d, _p(counts), counts.numel(), stream_ptr()), "moe_combine")


GATE_SILU, GATE_SIGMOID = 0, 1


def gated_head_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, weight_per_head: bool, act: int,
                    eps: float, out: torch.Tensor, num_heads: int, value_dim: int) -> None:
    """out = o / rms_head(o) * weight * act(gate): o fp32 [T, H*vd], gate [T, >=H*vd] (may be a column
    view), weight [vd] shared by the heads or [H*vd]."""
    require_cuda(o, gate, weight, out)
    _contig(o, "o"); _contig(out, "out"); _contig(weight, "weight")
    T = o.shape[0]
    if o.dtype != torch.float32 or o.shape != (T, num_heads * value_dim) or out.shape != o.shape:
        raise KernelError("gated_head_norm: o is fp32 [T, H*vd] and out has its shape")
    if gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] != o.shape[1] or gate.dtype != out.dtype:
        raise KernelError("gated_head_norm: gate is [T, H*vd] of out's dtype with unit column stride")
    if weight.numel() != (num_heads * value_dim if weight_per_head else value_dim):
        raise KernelError("gated_head_norm: weight size")
    check(L.core().ri_gated_head_norm(_p(o), _p(gate), gate.stride(0), _p(weight), dtype_code(weight.dtype),
                                      1 if weight_per_head else 0, int(act), float(eps), _p(out),
                                      dtype_code(out.dtype), T, num_heads, value_dim, stream_ptr()), "gated_head_norm")


ACT_GELU_ERF, ACT_TANH, ACT_GELU_TANH, ACT_RELU_SQUARED, ACT_SILU = 0, 1, 2, 3, 4


def activation(x: torch.Tensor, out: torch.Tensor, kind: int) -> None:
    require_cuda(x, out)
    _contig(x, "x"); _contig(out, "out")
    if x.shape != out.shape or x.dtype != out.dtype:
        raise KernelError("activation: out has x's shape and dtype")
    check(L.core().ri_activation(_p(x), _p(out), dtype_code(x.dtype), x.numel(), int(kind), stream_ptr()), "activation")


def activation_cols(x: torch.Tensor, kind: int) -> None:
    """x [rows, cols] with unit column stride (the leading columns of wider rows, say), in place."""
    require_cuda(x)
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("activation_cols: x is [rows, cols] with unit column stride")
    check(L.core().ri_activation_cols(_p(x), dtype_code(x.dtype), x.stride(0), x.shape[0], x.shape[1], int(kind),
                                      stream_ptr()), "activation_cols")


def scaled_sum(a: torch.Tensor, b: torch.Tensor, sa: float, sb: float, out: torch.Tensor) -> None:
    """out = sa * a + sb * b."""
    require_cuda(a, b, out)
    _contig(a, "a"); _contig(b, "b"); _contig(out, "out")
    if a.shape != b.shape or a.shape != out.shape or a.dtype != b.dtype or a.dtype != out.dtype:
        raise KernelError("scaled_sum: a, b and out share shape and dtype")
    check(L.core().ri_scaled_sum(_p(a), _p(b), float(sa), float(sb), _p(out), dtype_code(a.dtype), a.numel(),
                                 stream_ptr()), "scaled_sum")


_rows_checked = set()


def recurrent_state_rows(key_dim: int) -> int:
    """Rows a stored column of the recurrences' state has: the key size rounded up so that each of the
    lanes that share a column (4, 8, 16 or 32: as few as leave a lane at most 4 rows) holds a multiple
    of 4 rows.  The state of one request and head is [value_dim, rows] fp32; rows beyond key_dim stay zero."""
    lanes = 4 if key_dim <= 16 else 8 if key_dim <= 32 else 16 if key_dim <= 64 else 32
    per_lane = -(-(-(-key_dim // lanes)) // 4) * 4
    return lanes * per_lane


def _scan_common(state: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor,
                 T: int, H: int, dk: int, dv: int, what: str) -> None:
    _i32(cu_q, "cu_q"); _i32(state_slots, "state_slots")
    _contig(state, "state"); _contig(out, "out")
    rows = recurrent_state_rows(dk)
    if dk not in _rows_checked:                       # once per key size: host and kernel count alike
        kept = int(L.recurrent(dk).ri_recurrent_state_rows())
        if kept != rows:
            raise KernelError(f"{what}: the kernel stores {kept} rows a column, the host counts {rows}")
        _rows_checked.add(dk)
    if state.dtype != torch.float32 or state.dim() != 4 or tuple(state.shape[1:]) != (H, dv, rows):
        raise KernelError(f"{what}: state is fp32 [slots, {H}, {dv}, {rows}] (recurrent_state_rows({dk}) rows a column)")
    if out.dtype != torch.float32 or out.shape != (T, H * dv):
        raise KernelError(f"{what}: out is fp32 [T, H*dv]")


def _cols(t: torch.Tensor, T: int, n: int, dtype: torch.dtype, what: str) -> None:
    if t.dim() != 2 or t.shape != (T, n) or t.stride(1) != 1 or t.dtype != dtype:
        raise KernelError(f"{what} must be [{T}, {n}] {dtype} with unit column stride")


def gated_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, z_bias: Optional[torch.Tensor],
               q_scale: float, tau: float, out: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor,
               state_slots: torch.Tensor, entries: int, num_heads: int, key_dim: int, value_dim: int) -> None:
    """Gated linear attention over every entry's tokens in order, from and into state[slot]:
    S = diag(sigmoid(z + z_bias)^(1/tau)) S + k v^T, out = S^T (q * q_scale).  q, k [T, H*dk], v [T, H*dv]
    (column views allowed), z fp32 [T, H*dk]; state [slots, H, dv, recurrent_state_rows(dk)].  Two
    launches: the decays of all tokens at once (z is overwritten with them), then the walk (a step in
    which every entry brings one token, T == entries, goes to the kernel without staging)."""
    require_cuda(q, k, v, z, z_bias, out, state, cu_q, state_slots)
    T, H, dk, dv = q.shape[0], num_heads, key_dim, value_dim
    _scan_common(state, out, cu_q, state_slots, T, H, dk, dv, "gated_scan")
    _cols(q, T, H * dk, q.dtype, "gated_scan: q"); _cols(k, T, H * dk, q.dtype, "gated_scan: k")
    _cols(v, T, H * dv, q.dtype, "gated_scan: v"); _cols(z, T, H * dk, torch.float32, "gated_scan: z")
    _contig(z, "z")
    if z_bias is not None and z_bias.numel() != H * dk:
        raise KernelError("gated_scan: z_bias has H*dk elements")
    check(L.core().ri_gated_decay(_p(z), _p(z_bias), dtype_code(z_bias.dtype) if z_bias is not None else 0,
                                  1.0 / float(tau), T, H * dk, stream_ptr()), "gated_decay")
    check(L.recurrent(dk).ri_gated_scan(_p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(z), z.stride(0),
                                        dtype_code(q.dtype), float(q_scale), _p(out), _p(state), _p(cu_q),
                                        _p(state_slots), int(entries), H, dv, 1 if T == int(entries) else 0,
                                        stream_ptr()), "gated_scan")


def decay_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, q_scale: float,
               out: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, entries: int,
               num_heads: int, key_dim: int, value_dim: int) -> None:
    """Linear attention with decays that do not depend on the token, over every entry's tokens in order, from
    and into state[slot]: S = diag(decay) S + k v^T, out = S^T (q * q_scale).  `decay` fp32 [H*dk] (a head's
    one decay repeated over its key channels, or one per channel); the rest as `gated_scan`.  The walk is
    `gated_scan`'s: every token reads the same row of decays."""
    require_cuda(q, k, v, decay, out, state, cu_q, state_slots)
    T, H, dk, dv = q.shape[0], num_heads, key_dim, value_dim
    _scan_common(state, out, cu_q, state_slots, T, H, dk, dv, "decay_scan")
    _cols(q, T, H * dk, q.dtype, "decay_scan: q"); _cols(k, T, H * dk, q.dtype, "decay_scan: k")
    _cols(v, T, H * dv, q.dtype, "decay_scan: v")
    if decay.dtype != torch.float32 or decay.numel() != H * dk or not decay.is_contiguous():
        raise KernelError("decay_scan: decay is fp32 [H*dk]")
    check(L.recurrent(dk).ri_gated_scan(_p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(decay), 0,
                                        dtype_code(q.dtype), float(q_scale), _p(out), _p(state), _p(cu_q),
                                        _p(state_slots), int(entries), H, dv, 1 if T == int(entries) else 0,
                                        stream_ptr()), "decay_scan")


def delta_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, za: torch.Tensor, za_bias: Optional[torch.Tensor],
               zw: torch.Tensor, zw_bias: Optional[torch.Tensor], decay_rate: float, unit_eps: float,
               out: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, entries: int,
               num_heads: int, key_dim: int, value_dim: int) -> None:
    """Delta rule with a decay, over every entry's tokens in order, from and into state[slot]:
    S = diag(w) S - (a * u)(u^T S) + k v^T, out = S^T r, with u = k / sqrt(|k|^2 + unit_eps),
    w = exp(-decay_rate * sigmoid(zw + zw_bias)), a = sigmoid(za + za_bias).  zw is fp32 and is
    overwritten with the decays.  Two launches: w, u and a * u of all tokens at once, then the walk."""
    require_cuda(r, k, v, za, za_bias, zw, zw_bias, out, state, cu_q, state_slots)
    T, H, dk, dv = r.shape[0], num_heads, key_dim, value_dim
    _scan_common(state, out, cu_q, state_slots, T, H, dk, dv, "delta_scan")
    for t, n, what in ((r, H * dk, "r"), (k, H * dk, "k"), (v, H * dv, "v"), (za, H * dk, "za")):
        _cols(t, T, n, r.dtype, "delta_scan: " + what)
    _cols(zw, T, H * dk, torch.float32, "delta_scan: zw")
    _contig(zw, "zw")
    biases = [b for b in (za_bias, zw_bias) if b is not None]
    for b in biases:
        if b.numel() != H * dk or b.dtype != biases[0].dtype:
            raise KernelError("delta_scan: biases have H*dk elements and one dtype")
    unit = torch.empty((2, T, H * dk), dtype=torch.float32, device=r.device)      # u, a * u
    check(L.core().ri_delta_prepare(_p(k), k.stride(0), _p(za), za.stride(0), _p(za_bias), _p(zw), _p(zw_bias),
                                    dtype_code(r.dtype), dtype_code(biases[0].dtype) if biases else 0,
                                    float(decay_rate), float(unit_eps), _p(unit[0]), _p(unit[1]), T, H, dk,
                                    stream_ptr()), "delta_prepare")
    check(L.recurrent(dk).ri_delta_scan(_p(r), r.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(zw), _p(unit[0]),
                                        _p(unit[1]), H * dk, dtype_code(r.dtype), _p(out), _p(state), _p(cu_q),
                                        _p(state_slots), int(entries), H, dv, 1 if T == int(entries) else 0,
                                        stream_ptr()), "delta_scan")


# ------------------------------------------------- blocks that norm after the sum, and their mixers
def embed_scaled(ids: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor) -> None:
    """out[t,:] (fp32) = scale * table[ids[t],:]."""
    require_cuda(ids, table, out)
    _i32(ids, "ids"); _contig(table, "table"); _contig(out, "out")
    if out.dtype != torch.float32 or out.shape != (ids.numel(), table.shape[1]):
        raise KernelError(f"embed_scaled: out must be fp32 [{ids.numel()}, {table.shape[1]}]")
    check(L.core().ri_embed_scaled(_p(ids), _p(table), dtype_code(table.dtype), float(scale), _p(out), ids.numel(),
                                   table.shape[1], table.shape[0], stream_ptr()), "embed_scaled")


def round_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (fp32) rounded to out's dtype."""
    require_cuda(x, out)
    _contig(x, "x"); _contig(out, "out")
    if x.dtype != torch.float32 or x.shape != out.shape:
        raise KernelError("round_rows: x is fp32 and out has its shape")
    check(L.core().ri_round_rows(_p(x), _p(out), dtype_code(out.dtype), x.numel(), stream_ptr()), "round_rows")


def scale_add_norm(h: torch.Tensor, delta: Optional[torch.Tensor], bias: Optional[torch.Tensor], alpha: float,
                   weight: torch.Tensor, eps: float, act: Optional[torch.Tensor]) -> None:
    """h (fp32 [T,d]) <- weight * rms(alpha * h + delta + bias), in place; `act` (may be None) gets the new
    h rounded to its dtype.  delta fp32 or bf16; bias (may be None) has the weight's dtype."""
    require_cuda(h, delta, bias, weight, act)
    _contig(h, "h"); _contig(weight, "weight")
    T, d = h.shape
    if h.dtype != torch.float32 or weight.numel() != d:
        raise KernelError("scale_add_norm: the stream is fp32 and the weight has a row's size")
    if delta is not None and (delta.shape != h.shape or not delta.is_contiguous()):
        raise KernelError("scale_add_norm: delta has the stream's shape")
    if bias is not None and (bias.numel() != d or bias.dtype != weight.dtype or not bias.is_contiguous()):
        raise KernelError("scale_add_norm: bias has a row's size and the weight's dtype")
    if act is not None and (act.shape != h.shape or not act.is_contiguous()):
        raise KernelError("scale_add_norm: act has the stream's shape")
    check(L.core().ri_scale_add_norm(_p(h), _p(delta), dtype_code(delta.dtype) if delta is not None else 0, _p(bias),
                                     float(alpha), _p(weight), dtype_code(weight.dtype), float(eps), _p(act),
                                     dtype_code(act.dtype) if act is not None else 0, T, d, stream_ptr()),
          "scale_add_norm")


def row_norm_gate(o: torch.Tensor, gate: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                  out: torch.Tensor) -> None:
    """out = weight * o / rms(o) * sigmoid(gate), the root mean square over the whole row: o fp32 [T, n],
    gate [T, n] (may be a column view; None: no gate), weight [n]."""
    require_cuda(o, gate, weight, out)
    _contig(o, "o"); _contig(out, "out"); _contig(weight, "weight")
    if o.dtype != torch.float32 or o.dim() != 2 or out.shape != o.shape or weight.numel() != o.shape[1]:
        raise KernelError("row_norm_gate: o is fp32 [T, n], out has its shape, weight a row's size")
    if gate is not None and (gate.shape != o.shape or gate.stride(1) != 1):
        raise KernelError("row_norm_gate: gate is [T, n] with unit column stride")
    check(L.core().ri_row_norm_gate(_p(o), _p(gate), dtype_code(gate.dtype) if gate is not None else 0,
                                    gate.stride(0) if gate is not None else 0, _p(weight), dtype_code(weight.dtype),
                                    float(eps), _p(out), dtype_code(out.dtype), o.shape[0], o.shape[1], stream_ptr()),
          "row_norm_gate")


def diff_combine(a: torch.Tensor, lam: float, out_scale: float, eps: float, gate: Optional[torch.Tensor],
                 out: torch.Tensor, num_heads: int, value_dim: int) -> None:
    """a fp32 [T, H*2*vd], a head's two attention maps side by side: out[t, h] = out_scale * o / rms(o) *
    sigmoid(gate[t, h]) with o = a1 - lam * a2 and the root mean square over the head's vd values."""
    require_cuda(a, gate, out)
    _contig(a, "a"); _contig(out, "out")
    T = a.shape[0]
    if a.dtype != torch.float32 or a.shape != (T, num_heads * 2 * value_dim) or out.shape != (T, num_heads * value_dim):
        raise KernelError("diff_combine: a is fp32 [T, H*2*vd], out [T, H*vd]")
    if gate is not None and (gate.shape != out.shape or gate.stride(1) != 1):
        raise KernelError("diff_combine: gate is [T, H*vd] with unit column stride")
    check(L.core().ri_diff_combine(_p(a), float(lam), float(out_scale), float(eps), _p(gate),
                                   dtype_code(gate.dtype) if gate is not None else 0,
                                   gate.stride(0) if gate is not None else 0, _p(out), dtype_code(out.dtype), T,
                                   num_heads, value_dim, stream_ptr()), "diff_combine")


def latent_prepare(proj: torch.Tensor, c_weight: torch.Tensor, eps: float, positions: torch.Tensor,
                   cos: torch.Tensor, sin: torch.Tensor, slot_of_token: Optional[torch.Tensor],
                   cache: Optional[torch.Tensor], q_plain: torch.Tensor, q_full: torch.Tensor, num_heads: int,
                   head_dim: int, rot_dim: int, rank: int, low: Optional[torch.Tensor] = None,
                   interleaved: bool = True) -> None:
    """proj [T, H*(d+r) + rank + r]: every head's plain (d) and rotated (r) query channels, then the low-rank
    vector and the key part all heads share.  Writes the plain query parts into q_plain [T, H*d], the rotated
    ones into the last r channels of every head of q_full [T, H*(rank+r)], and the cache row of the token
    (the low-rank vector normed with c_weight, then the rotated shared key part) at slot_of_token[t].
    With `low` [T, rank + r] (of proj's dtype, unit column stride) proj holds the queries only, [T, H*(d+r)].
    `interleaved`: the rotary pairs are channels (2i, 2i+1); else (i, i + r/2)."""
    require_cuda(proj, c_weight, positions, cos, sin, slot_of_token, cache, q_plain, q_full, low)
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token")
    T, H, d, r = proj.shape[0], num_heads, head_dim, rot_dim
    cols = H * (d + r) + (0 if low is not None else rank + r)
    if proj.stride(1) != 1 or proj.shape[1] != cols:
        raise KernelError(f"latent_prepare: proj is [T, {cols}] with unit column stride")
    if low is not None and (low.dtype != proj.dtype or low.shape != (T, rank + r) or low.stride(1) != 1):
        raise KernelError(f"latent_prepare: low is [T, {rank + r}] of proj's dtype with unit column stride")
    _contig(q_plain, "q_plain"); _contig(q_full, "q_full"); _contig(c_weight, "c_weight")
    if q_plain.shape != (T, H * d) or q_full.shape != (T, H * (rank + r)) or q_plain.dtype != q_full.dtype:
        raise KernelError("latent_prepare: q_plain is [T, H*d], q_full [T, H*(rank+r)], of one dtype")
    if c_weight.numel() != rank:
        raise KernelError("latent_prepare: the norm weight has the low-rank vector's size")
    for t in (cos, sin):
        if t.dtype != torch.float32 or t.shape[1] != r // 2 or not t.is_contiguous():
            raise KernelError("latent_prepare: cos/sin are fp32 [positions, r/2]")
    if cache is not None:
        _contig(cache, "cache")
        if cache.dtype != q_full.dtype or cache.dim() != 2 or cache.shape[1] % (rank + r):
            raise KernelError("latent_prepare: the cache is [pages, page*(rank+r)] of q's dtype")
    check(L.core().ri_latent_prepare(_p(proj), dtype_code(proj.dtype), proj.stride(0), _p(c_weight),
                                     dtype_code(c_weight.dtype), float(eps), _p(positions), _p(cos), _p(sin),
                                     _p(slot_of_token), _p(cache), _p(q_plain), _p(q_full), dtype_code(q_full.dtype),
                                     T, H, d, r, rank, _p(low), low.stride(0) if low is not None else 0,
                                     1 if interleaved else 0, stream_ptr()), "latent_prepare")


def bias_rows(x: torch.Tensor, bias: torch.Tensor) -> None:
    """x [T, n] += bias [n], in place."""
    require_cuda(x, bias)
    _contig(x, "x"); _contig(bias, "bias")
    if x.dim() != 2 or bias.numel() != x.shape[1]:
        raise KernelError("bias_rows: bias has a row's size")
    check(L.core().ri_bias_rows(_p(x), dtype_code(x.dtype), _p(bias), dtype_code(bias.dtype), x.shape[0], x.shape[1],
                                stream_ptr()), "bias_rows")


def _attention_args(q, out, cache, block_table, cu_q, kv_len, num_heads, num_kv_heads, head_dim):
    require_cuda(q, out, cache, block_table, cu_q, kv_len)
    for t, n in ((block_table, "block_table"), (cu_q, "cu_q"), (kv_len, "kv_len")):
        _i32(t, n)
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("tensor-core attention takes bfloat16 q, out and cache")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.stride(0) % 8 or q.data_ptr() % 16 or out.stride(0) % 2:
        raise KernelError("tensor-core attention: q rows must be 16-byte aligned with unit column stride")
    _contig(cache, "cache")
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
        raise KernelError("attention: cache must be [pages, 2, Hkv, page, head_dim]")
    if num_heads % num_kv_heads:
        raise KernelError("attention: heads must be a multiple of kv heads")


def mma_tokens_per_tile(num_heads: int, num_kv_heads: int) -> int:
    """Query tokens one prefill CTA of the tensor-core kernel covers for this grouping."""
    return 64 // min(num_heads // num_kv_heads, 64)


def attention_prefill_bf16(q, out, cache, block_table, cu_q, kv_len, tile_entry, tile_tok0,
                           num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                           window: Optional[int], block: Optional[int] = None, precise: bool = False,
                           sink: bool = False) -> None:
    """Tiles are (entry, first token) pairs of `mma_tokens_per_tile` tokens each.  `block`: a query
    sees only the keys of its own block of that many positions.  `precise`: the softmax weights go
    into the product with the values in full fp32 (as three bf16 pieces) instead of rounded to bf16."""
    _attention_args(q, out, cache, block_table, cu_q, kv_len, num_heads, num_kv_heads, head_dim)
    require_cuda(tile_entry, tile_tok0)
    _i32(tile_entry, "tile_entry"); _i32(tile_tok0, "tile_tok0")
    lib = L.attention_mma(head_dim)
    check(lib.ri_attention_prefill_bf16(_p(q), q.stride(0), _p(out), out.stride(0), _p(cache), _p(block_table),
                                        block_table.stride(0), _p(cu_q), _p(kv_len), _p(tile_entry),
                                        _p(tile_tok0), tile_entry.numel(), num_heads, num_kv_heads,
                                        cache.shape[3], float(scale), int(window) if window else 0,
                                        int(block) if block else 0, 1 if precise else 0, 1 if sink else 0,
                                        stream_ptr()), "attention_prefill_bf16")


def tc_attention_supports(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes this geometry."""
    if head_dim not in (64, 128):
        return False
    return bool(L.attention_tc(head_dim).ri_attention_tc_supports(num_heads, num_kv_heads, page_size))


def tc_tokens_per_tile(num_heads: int, num_kv_heads: int) -> int:
    return 128 // (num_heads // num_kv_heads)


def attention_prefill_tc(q, out, cache, block_table, cu_q, kv_len, tile_entry, tile_tok0,
                         num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                         window: Optional[int]) -> None:
    """Prompt attention on tcgen05 tensor cores with TMA page fetches.  Tiles are (entry,
    first token) pairs of `tc_tokens_per_tile` tokens each."""
    _attention_args(q, out, cache, block_table, cu_q, kv_len, num_heads, num_kv_heads, head_dim)
    require_cuda(tile_entry, tile_tok0)
    _i32(tile_entry, "tile_entry"); _i32(tile_tok0, "tile_tok0")
    if out.stride(0) % 8 or out.data_ptr() % 16 or cache.data_ptr() % 16:
        raise KernelError("attention_prefill_tc: out rows and the cache must be 16-byte aligned")
    err = gemm_tc_state(q.device)[2]
    lib = L.attention_tc(head_dim)
    check(lib.ri_attention_prefill_tc(_p(q), q.stride(0), _p(out), out.stride(0), _p(cache), cache.shape[0],
                                      _p(block_table), block_table.stride(0), _p(cu_q), _p(kv_len),
                                      _p(tile_entry), _p(tile_tok0), tile_entry.numel(), num_heads,
                                      num_kv_heads, cache.shape[3], float(scale), int(window) if window else 0,
                                      _p(err), stream_ptr()), "attention_prefill_tc")


def decode_scratch_floats(entries: int, num_heads: int, head_dim: int, splits: int):
    return entries * num_heads * splits * head_dim, entries * num_heads * splits


def attention_decode_bf16(q, out, cache, block_table, cu_q, kv_len, entry_list: Optional[torch.Tensor],
                          n_entries: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                          window: Optional[int], splits: int, part_o: Optional[torch.Tensor],
                          part_lse: Optional[torch.Tensor], by_tma: bool = True, merge: bool = True) -> None:
    """Entries of one token each (entry_list: their indices, None = 0..n-1); `splits` > 1
    cuts each entry's keys into that many ranges whose partial results go through
    part_o / part_lse (fp32 scratch).  Head sizes 64 and 128 with pages of 8, 16, 32 or a
    multiple of 64 keys fetch keys and values by TMA unless `by_tma` is False.  With `merge`
    False (and several ranges) the ranges are not merged: `out` stays unwritten and the caller
    reads part_o [entries, Hq, splits, hd] and part_lse [entries, Hq, splits] itself."""
    _attention_args(q, out, cache, block_table, cu_q, kv_len, num_heads, num_kv_heads, head_dim)
    require_cuda(entry_list, part_o, part_lse)
    _i32(entry_list, "entry_list")
    if splits > 1:
        need_o, need_l = decode_scratch_floats(n_entries, num_heads, head_dim, splits)
        if part_o is None or part_lse is None or part_o.dtype != torch.float32 or \
                part_lse.dtype != torch.float32 or part_o.numel() < need_o or part_lse.numel() < need_l:
            raise KernelError(f"attention_decode: scratch must hold {need_o} and {need_l} fp32")
    lib = L.attention_mma(head_dim)
    check(lib.ri_attention_decode_bf16(_p(q), q.stride(0), _p(out), out.stride(0), _p(cache), _p(block_table),
                                       block_table.stride(0), _p(cu_q), _p(kv_len), _p(entry_list), n_entries,
                                       num_heads, num_kv_heads, cache.shape[3], float(scale),
                                       int(window) if window else 0, int(splits), _p(part_o), _p(part_lse),
                                       cache.shape[0] if by_tma else 0, _p(gemm_tc_state(q.device)[2]),
                                       1 if merge else 0, stream_ptr()), "attention_decode_bf16",
          2 if splits > 1 and merge else 1)


_argmax_state = {}


def argmax_state(device: torch.device, rows: int) -> torch.Tensor:
    """Zeroed scratch of the argmax kernel for up to `rows` rows: int64 [2 * rows], the
    merged keys followed by the arrival counters.  The kernel leaves it zero."""
    return torch.zeros(2 * rows, dtype=torch.int64, device=device)


def argmax(logits: torch.Tensor, out: torch.Tensor, state: Optional[torch.Tensor] = None) -> None:
    """out[r] = index of the largest logit of row r, the lowest index among equals."""
    require_cuda(logits, out, state)
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32:
        raise KernelError("argmax: logits fp32 [R,V], out int32 [R]")
    R = logits.shape[0]
    if state is None:
        key = (logits.device, torch.cuda.current_stream().cuda_stream)
        state = _argmax_state.get(key)
        if state is None or state.numel() < 2 * R:
            state = argmax_state(logits.device, max(R, 64))
            _argmax_state[key] = state
    if state.dtype != torch.int64 or state.numel() < 2 * R:
        raise KernelError(f"argmax: state must be int64 [{2 * R}]")
    check(L.core().ri_argmax(_p(logits), logits.stride(0), R, logits.shape[1], _p(out),
                             state.data_ptr(), state.data_ptr() + 8 * (state.numel() // 2),
                             stream_ptr()), "argmax")


def decode_feedback(sampled: torch.Tensor, state_slots: torch.Tensor, slot_state: torch.Tensor,
                    eos_ids: Optional[torch.Tensor], result: torch.Tensor,
                    token_feed: Optional[torch.Tensor]) -> None:
    """Per row of a decode step: count the chosen token in slot_state[slot] = {generated,
    max_tokens, ignore_eos, last_token}, write result = [tokens | stop flags] (int32
    [2 * rows]) and copy the token to `token_feed`, the next step's input ids."""
    require_cuda(sampled, state_slots, slot_state, eos_ids, result, token_feed)
    rows = sampled.numel()
    for t, n in ((sampled, "sampled"), (state_slots, "state_slots"), (slot_state, "slot_state"),
                 (eos_ids, "eos_ids"), (result, "result"), (token_feed, "token_feed")):
        _i32(t, n)
    if state_slots.numel() < rows or result.numel() < 2 * rows or slot_state.dim() != 2 or slot_state.shape[1] != 4 \
            or not slot_state.is_contiguous() or (token_feed is not None and token_feed.numel() < rows):
        raise KernelError("decode_feedback: sizes")
    check(L.core().ri_decode_feedback(_p(sampled), _p(state_slots), rows, _p(slot_state), _p(eos_ids),
                                      0 if eos_ids is None else eos_ids.numel(), _p(result), _p(token_feed),
                                      stream_ptr()), "decode_feedback")


def sample(logits: torch.Tensor, scratch: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, min_p: torch.Tensor, draw: torch.Tensor, out: torch.Tensor,
           by_sorting: bool = False) -> None:
    """out[r] = the token drawn for row r: logit / temperature, top-k, min-p, top-p, then the token at
    which the running weight passes draw[r] * (kept weight).  `by_sorting` runs the kernel that sorts
    every row whole (the slow statement the bucketed kernel falls back to)."""
    require_cuda(logits, scratch, temperature, top_k, top_p, min_p, draw, out)
    R, V = logits.shape
    vpad = 1 << max(1, (V - 1).bit_length())
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits fp32 [R,V]")
    if scratch.dtype != torch.int64 or scratch.numel() < R * vpad + R:
        raise KernelError(f"sample: scratch must hold {R * vpad + R} int64")
    if (temperature.dtype, top_k.dtype, top_p.dtype, min_p.dtype, draw.dtype, out.dtype) != \
            (torch.float32, torch.int32, torch.float32, torch.float32, torch.float64, torch.int32):
        raise KernelError("sample: parameter dtypes")
    fn = L.core().ri_sample_by_sorting if by_sorting else L.core().ri_sample
    check(fn(_p(logits), logits.stride(0), R, V, vpad, _p(scratch), _p(temperature),
             _p(top_k), _p(top_p), _p(min_p), _p(draw), _p(out), stream_ptr()), "sample", 1 if by_sorting else 2)


def sample_scratch_elems(rows: int, vocab: int) -> int:
    """int64 words of scratch for `rows` rows: room for the rows that are sorted whole, and a flag a row."""
    return rows * (1 << max(1, (vocab - 1).bit_length())) + rows
