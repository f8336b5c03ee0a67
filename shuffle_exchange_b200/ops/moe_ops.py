"""Token routing primitives for mixture-of-experts layers (training and inference).

Kernels: ``csrc/moe_ragged.cu`` — ``sxb_top_k_gating`` (softmax over all experts + top-k + per-expert arrival order),
``sxb_moe_scatter`` (dropless grouping of token rows by expert), ``sxb_moe_gather`` (score-weighted combine) and its
backward.  They replace the dense one-hot einsum dispatch/combine of the reference (``moe/sharded_moe.py:609-610,670``:
O(S·E·C·M) FLOPs and memory) and are the same operations as its inference kernels
(``inference/v2/kernels/ragged_ops/{top_k_gating,moe_scatter,moe_gather}``).  Each op has a PyTorch branch with the
same semantics, used on CPU and as the oracle in tests.
"""
from __future__ import annotations

from typing import Tuple

import torch

from ..native import lib as _lib

_lib.register({
    "sxb_top_k_gating": "ppppp" "iiii" "i" "p",
    "sxb_grouped_top_k_gating": "pppppp" "iiiii" "f" "p",
    "sxb_copy_group_rows": "ppp" "iii" "l" "p",
    "sxb_moe_scatter": "ppppppp" "iiiii" "p",
    "sxb_moe_scatter_scaled": "pppppppp" "iiiii" "p",
    "sxb_moe_gather": "pppp" "iii" "p",
    "sxb_moe_gather_bwd": "pppppp" "iii" "p",
})


def top_k_gating(logits: torch.Tensor, top_k: int, renormalize: bool = True, score_function: str = "softmax",
                 correction: torch.Tensor = None, n_groups: int = 1, keep_groups: int = 1, scale: float = 1.0):
    """``logits`` [T, E] -> ``(scores fp32 [T,K], assignments int32 [T,K], offsets int32 [T,K], counts int32 [E])``.

    ``score_function`` ``"softmax"``: scores are the softmax over all experts; ``"sigmoid"``: every expert is scored on
    its own with ``sigmoid(logit)``.  The ``top_k`` largest win either way; ``renormalize`` divides them by their sum.

    Group-limited choice (softmax scores only; taken when ``correction`` is given, ``n_groups > 1`` or ``scale != 1``):
    the winners are the ``top_k`` largest ``score + correction`` (``correction`` fp32 ``[E]``) among the experts of the
    ``keep_groups`` groups -- of ``n_groups`` equal contiguous blocks of experts -- whose best ``score + correction``
    is largest; the returned scores are the winners' plain scores normalised by their total (1e-20 added), times ``scale``.

    ``offsets[t,k]`` is the arrival index of token ``t`` inside expert ``assignments[t,k]`` (a permutation of
    ``range(counts[e])`` per expert; on CUDA the order is nondeterministic, on CPU it is token order)."""
    T, E = logits.shape
    dev = logits.device
    if score_function not in ("softmax", "sigmoid"):
        raise ValueError(f"unknown score function {score_function!r}")
    scores = torch.empty(T, top_k, dtype=torch.float32, device=dev)
    assign = torch.empty(T, top_k, dtype=torch.int32, device=dev)
    offsets = torch.empty(T, top_k, dtype=torch.int32, device=dev)
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    grouped = correction is not None or n_groups > 1 or scale != 1.0
    if grouped:
        if score_function != "softmax":
            raise ValueError("the group-limited choice scores with the softmax over all experts")
        if E % n_groups or not 1 <= keep_groups <= n_groups or top_k > keep_groups * (E // n_groups):
            raise ValueError(f"cannot choose {top_k} of {E} experts in {keep_groups} of {n_groups} groups")
    if grouped and logits.is_cuda:
        logits = logits.float().contiguous()
        corr = None if correction is None else correction.float().contiguous()
        _lib.call("sxb_grouped_top_k_gating", logits.data_ptr(), _lib.ptr(corr), scores.data_ptr(), assign.data_ptr(),
                  offsets.data_ptr(), counts.data_ptr(), T, E, top_k, int(n_groups), int(keep_groups), float(scale),
                  _lib.stream_ptr())
        return scores, assign, offsets, counts
    if grouped:
        probs = torch.softmax(logits.float(), dim=-1)
        choice = probs if correction is None else probs + correction.float()
        if keep_groups < n_groups:
            per = E // n_groups
            best = choice.view(T, n_groups, per).max(dim=-1).values
            kept = torch.zeros(T, n_groups, dtype=torch.bool, device=dev)
            kept.scatter_(1, torch.topk(best, keep_groups, dim=-1).indices, True)
            choice = choice.masked_fill(~kept.repeat_interleave(per, dim=1), float("-inf"))
        a = torch.topk(choice, top_k, dim=-1).indices
        s = probs.gather(1, a)
        s = s / (s.sum(dim=-1, keepdim=True) + 1e-20) * scale
        flat = a.reshape(-1)
        onehot = torch.nn.functional.one_hot(flat, E)
        order = (torch.cumsum(onehot, dim=0) - 1).gather(1, flat[:, None]).squeeze(1)
        scores.copy_(s)
        assign.copy_(a.to(torch.int32))
        offsets.copy_(order.view(T, top_k).to(torch.int32))
        counts.copy_(onehot.sum(0).to(torch.int32))
        return scores, assign, offsets, counts
    if logits.is_cuda:
        logits = logits.contiguous()
        _lib.call("sxb_top_k_gating", logits.data_ptr(), scores.data_ptr(), assign.data_ptr(), offsets.data_ptr(),
                  counts.data_ptr(), T, E, top_k, int(bool(renormalize)) | (2 if score_function == "sigmoid" else 0),
                  _lib.dtype_code(logits.dtype), _lib.stream_ptr())
        return scores, assign, offsets, counts
    probs = torch.sigmoid(logits.float()) if score_function == "sigmoid" else torch.softmax(logits.float(), dim=-1)
    s, a = torch.topk(probs, top_k, dim=-1)
    if renormalize:
        s = s / s.sum(dim=-1, keepdim=True)
    flat = a.reshape(-1)
    onehot = torch.nn.functional.one_hot(flat, E)
    order = (torch.cumsum(onehot, dim=0) - 1).gather(1, flat[:, None]).squeeze(1)
    scores.copy_(s)
    assign.copy_(a.to(torch.int32))
    offsets.copy_(order.view(T, top_k).to(torch.int32))
    counts.copy_(onehot.sum(0).to(torch.int32))
    return scores, assign, offsets, counts


def _scatter_fwd(x, assign, offsets, counts):
    T, H = x.shape
    K = assign.shape[1]
    E = counts.shape[0]
    moe_in = torch.empty(T * K, H, dtype=x.dtype, device=x.device)
    cumsum = torch.empty(E, dtype=torch.int64, device=x.device)
    slots = torch.empty(T, K, dtype=torch.int32, device=x.device)
    if x.is_cuda:
        x = x.contiguous()
        if (H * x.element_size()) % 16 and x.dtype in (torch.bfloat16, torch.float32):
            # rows that are not whole 16-byte words: the element-wise form of the copy, with unit weights
            ones = torch.ones(T, K, dtype=torch.float32, device=x.device)
            _lib.call("sxb_moe_scatter_scaled", x.data_ptr(), ones.data_ptr(), moe_in.data_ptr(), assign.data_ptr(),
                      offsets.data_ptr(), counts.data_ptr(), cumsum.data_ptr(), slots.data_ptr(), T, E, K, H,
                      _lib.dtype_code(x.dtype), _lib.stream_ptr())
            return moe_in, cumsum, slots
        _lib.call("sxb_moe_scatter", x.data_ptr(), moe_in.data_ptr(), assign.data_ptr(), offsets.data_ptr(),
                  counts.data_ptr(), cumsum.data_ptr(), slots.data_ptr(), T, E, K, H, x.element_size(), _lib.stream_ptr())
        return moe_in, cumsum, slots
    cumsum.copy_(torch.cumsum(counts.long(), 0))
    base = torch.cat([cumsum.new_zeros(1), cumsum[:-1]])
    sl = base[assign.long()] + offsets.long()
    slots.copy_(sl.to(torch.int32))
    moe_in[sl.reshape(-1)] = x.repeat_interleave(K, dim=0)
    return moe_in, cumsum, slots


def _gather_fwd(moe_out, scores, slots):
    T, K = slots.shape
    H = moe_out.shape[1]
    if moe_out.is_cuda and moe_out.dtype == torch.bfloat16 and H % 8 == 0:      # rows of whole 16-byte words
        out = torch.empty(T, H, dtype=moe_out.dtype, device=moe_out.device)
        _lib.call("sxb_moe_gather", moe_out.data_ptr(), out.data_ptr(), None if scores is None else scores.data_ptr(),
                  slots.data_ptr(), T, K, H, _lib.stream_ptr())
        return out
    rows = moe_out[slots.long().reshape(-1)].view(T, K, H).float()
    if scores is not None:
        rows = rows * scores[:, :, None]
    return rows.sum(1).to(moe_out.dtype)


class _MoEScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, assign, offsets, counts):
        moe_in, cumsum, slots = _scatter_fwd(x, assign, offsets, counts)
        ctx.save_for_backward(slots)
        ctx.mark_non_differentiable(cumsum, slots)
        return moe_in, cumsum, slots

    @staticmethod
    def backward(ctx, d_moe_in, _c, _s):
        slots, = ctx.saved_tensors
        return _gather_fwd(d_moe_in.contiguous(), None, slots), None, None, None


class _MoEGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, moe_out, scores, slots):
        ctx.save_for_backward(moe_out, scores, slots)
        return _gather_fwd(moe_out, scores, slots)

    @staticmethod
    def backward(ctx, d_out):
        moe_out, scores, slots = ctx.saved_tensors
        T, K = slots.shape
        H = moe_out.shape[1]
        d_out = d_out.contiguous()
        if moe_out.is_cuda and moe_out.dtype == torch.bfloat16:
            d_moe = torch.empty_like(moe_out)
            d_scores = torch.empty(T, K, dtype=torch.float32, device=moe_out.device)
            _lib.call("sxb_moe_gather_bwd", d_out.data_ptr(), moe_out.data_ptr(), scores.data_ptr(), slots.data_ptr(),
                      d_moe.data_ptr(), d_scores.data_ptr(), T, K, H, _lib.stream_ptr())
            return d_moe, d_scores, None
        sl = slots.long().reshape(-1)
        d_moe = torch.zeros_like(moe_out)
        d_moe[sl] = (d_out.float()[:, None, :] * scores[:, :, None]).reshape(T * K, H).to(moe_out.dtype)
        d_scores = (moe_out[sl].view(T, K, H).float() * d_out.float()[:, None, :]).sum(-1)
        return d_moe, d_scores, None


def moe_scatter(x: torch.Tensor, assign: torch.Tensor, offsets: torch.Tensor, counts: torch.Tensor):
    """``x`` [T, H] -> ``(moe_input [T*K, H] grouped by expert, expert_cumsum int64 [E], mapped_slots int32 [T, K])``."""
    return _MoEScatter.apply(x, assign, offsets, counts)


def moe_gather(moe_output: torch.Tensor, scores: torch.Tensor, mapped_slots: torch.Tensor) -> torch.Tensor:
    """``out[t] = sum_k scores[t,k] * moe_output[mapped_slots[t,k]]`` (differentiable in both tensor arguments)."""
    return _MoEGather.apply(moe_output, scores, mapped_slots)


@torch.no_grad()
def moe_scatter_scaled(x: torch.Tensor, scores: torch.Tensor, assign: torch.Tensor, offsets: torch.Tensor,
                       counts: torch.Tensor):
    """:func:`moe_scatter` for layers whose routing weight multiplies the expert's INPUT: row ``(t, k)`` of the grouped
    input is ``x[t] * scores[t, k]`` (product in fp32, rounded once to ``x.dtype``).  Inference only; bf16 or fp32 rows
    of any width."""
    T, H = x.shape
    K, E = assign.shape[1], counts.shape[0]
    if x.is_cuda:
        x = x.contiguous()
        moe_in = torch.empty(T * K, H, dtype=x.dtype, device=x.device)
        cumsum = torch.empty(E, dtype=torch.int64, device=x.device)
        slots = torch.empty(T, K, dtype=torch.int32, device=x.device)
        _lib.call("sxb_moe_scatter_scaled", x.data_ptr(), scores.data_ptr(), moe_in.data_ptr(), assign.data_ptr(),
                  offsets.data_ptr(), counts.data_ptr(), cumsum.data_ptr(), slots.data_ptr(), T, E, K, H,
                  _lib.dtype_code(x.dtype), _lib.stream_ptr())
        return moe_in, cumsum, slots
    moe_in, cumsum, slots = _scatter_fwd(x, assign, offsets, counts)
    scaled = (x.float()[:, None, :] * scores[:, :, None]).to(x.dtype).reshape(T * K, H)
    moe_in[slots.long().reshape(-1)] = scaled
    return moe_in, cumsum, slots


def copy_group_rows_(dst: torch.Tensor, src: torch.Tensor, offsets: torch.Tensor, g_lo: int, g_hi: int) -> torch.Tensor:
    """``dst[offsets[g_lo] : offsets[g_hi]] = src[the same rows]`` for expert-sorted row buffers whose group offsets
    (int32, ``[groups + 1]``) live on the device: experts that hand their input on unchanged, without a host read."""
    if g_hi <= g_lo:
        return dst
    if src.is_cuda:
        if offsets.dtype != torch.int32 or not src.is_contiguous() or not dst.is_contiguous() or src.dtype != dst.dtype \
                or src.shape[1] != dst.shape[1]:
            raise ValueError("expected contiguous row buffers of one shape and dtype and int32 offsets")
        _lib.call("sxb_copy_group_rows", src.data_ptr(), dst.data_ptr(), offsets.data_ptr(), int(g_lo), int(g_hi),
                  src.shape[1] * src.element_size(), min(src.shape[0], dst.shape[0]), _lib.stream_ptr())
        return dst
    lo, hi = int(offsets[g_lo]), int(offsets[g_hi])
    dst[lo:hi] = src[lo:hi]
    return dst
