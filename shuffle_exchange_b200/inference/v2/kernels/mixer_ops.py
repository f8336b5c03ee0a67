"""Python entry points of the ragged-batch kernels for hybrid layer stacks (``csrc/seq_mixers.cu``): fp32 residual
stream with pre- and post-norms, chunk-local attention with a sink logit, short causal convolutions with carried inputs,
and the linear recurrences of the gated delta rule and of state-space duality.

As in ``ragged_ops``, every wrapper has a PyTorch branch with identical semantics (CPU execution and test oracle of the
kernels); CUDA tensors always take the kernel.  ``seq_info`` is int32 ``[n_seqs, 4]`` = (first row of the sequence in
the batch, rows, tokens already seen, state slot); activations are bf16 or fp32 (``x.dtype``), everything the norms,
softmax and recurrences touch is fp32.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ....native import lib as _lib

_lib.register({
    "sxb_embed_sinusoid": "pppp" "ii" "ff" "i" "p",
    "sxb_resid_norm_step": "pppppp" "l" "i" "ff" "i" "p" "f" "p",
    "sxb_qk_norm_append": "p" "l" "ppppppp" "iiiiiii" "f" "ii" "p",
    "sxb_qkv_filter_norm_append": "p" "l" "ppppppppppp" "iiiiiiii" "f" "i" "f" "i" "i" "p",
    "sxb_sink_attention": "pppppppp" "iiiiiii" "f" "iiii" "p" "i" "p" "l" "i" "p",
    "sxb_sink_attention_atoms": "pppppp" "ii" "p" "iiiiii" "f" "iiii" "p" "i" "p" "l" "i" "p",
    "sxb_conv_silu": "p" "l" "pppppp" "iii" "i" "p",
    "sxb_conv_state_update": "p" "l" "pp" "iii" "i" "p",
    "sxb_unit_norm_heads": "p" "l" "iii" "ff" "i" "p",
    "sxb_recurrence_gates": "pp" "l" "pppp" "iii" "i" "p",
    "sxb_linear_recurrence": "pp" "l" "p" "l" "pppppp" "iiiiii" "i" "p",
    "sxb_group_norm_gate": "pp" "l" "p" "i" "p" "iii" "f" "i" "i" "p",
    "sxb_gated_act_rows": "pp" "l" "ii" "i" "f" "p",
    "sxb_conv_residual": "pppppp" "iii" "i" "p",
    "sxb_post_norm_mix": "pppppp" "l" "i" "pp" "l" "i" "f" "i" "p",
    "sxb_rms_scale_rows": "pppp" "ii" "f" "i" "p",
    "sxb_rms_norm_slice": "p" "l" "pp" "ii" "f" "i" "p",
    "sxb_bias_act_rows": "ppp" "l" "ii" "i" "p",
    "sxb_latent_qk_prepare": "p" "l" "p" "ll" "p" "l" "ppppppp" "iii" "iiiii" "f" "i" "f" "p",
    "sxb_mlstm_prepare": "p" "l" "p" "iiii" "f" "i" "p",
    "sxb_mlstm_gate_scan": "pp" "l" "pp" "f" "ppppp" "iii" "i" "p",
    "sxb_mlstm_output": "ppp" "l" "pp" "iii" "f" "i" "p",
    "sxb_side_gate": "p" "l" "p" "l" "pp" "iiii" "i" "p",
    "sxb_scale_softcap": "p" "l" "ff" "p",
    "sxb_row_gate_add": "ppp" "l" "l" "i" "i" "p",
    "sxb_router_logits": "p" "l" "ppp" "iii" "i" "p",
    "sxb_channel_decay_gates": "p" "l" "p" "l" "pppp" "iii" "i" "p",
    "sxb_sigmoid_gate_rows": "pp" "l" "l" "ii" "i" "p",
    "sxb_power_norm_act": "pppp" "l" "i" "f" "i" "p",
})

_ACTS = {"identity": 0, "relu": 1, "gelu": 2, "silu": 3, "relu_sq": 4, "clamped_swish": 5}


def _dt(t: torch.Tensor) -> int:
    return _lib.dtype_code(t.dtype)


def _rows(t: torch.Tensor) -> torch.Tensor:
    """2-D view with unit inner stride (row pitch may exceed the width: column slices of a fused projection)."""
    if t.stride(-1) != 1:
        raise ValueError("expected unit inner stride")
    return t


# ------------------------------------------------------------------------------------------------ embedding
def embed_sinusoid(ids: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, scale: float,
                   base: Optional[float] = 10000.0) -> torch.Tensor:
    """fp32 ``[T, width]``: ``table[ids] * scale + p`` with ``p[2i] = sin(pos * base^(-2i/width))``, ``p[2i+1] = cos``;
    ``base`` None: no position vector."""
    T, W = ids.numel(), table.shape[1]
    if table.is_cuda:
        out = torch.empty(T, W, dtype=torch.float32, device=table.device)
        _lib.call("sxb_embed_sinusoid", ids.data_ptr(), positions.data_ptr(), table.data_ptr(), out.data_ptr(), T, W,
                  float(scale), 0.0 if base is None else float(base), _dt(table), _lib.stream_ptr())
        return out
    if base is None:
        return table[ids.long()].float() * scale
    i = torch.arange(W, device=table.device) // 2
    freq = torch.exp2(-(2.0 * i.float() / W) * math.log2(base))
    ang = positions.float()[:, None] * freq[None, :]
    pe = torch.where(torch.arange(W, device=table.device) % 2 == 1, ang.cos(), ang.sin())
    return table[ids.long()].float() * scale + pe


# ------------------------------------------------------------------------------------------------ residual + norms
def _rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def resid_norm_step(resid: torch.Tensor, y: Optional[torch.Tensor], w_post: Optional[torch.Tensor],
                    extra: Optional[torch.Tensor], w_pre: Optional[torch.Tensor], eps: float,
                    out_dtype: torch.dtype, mult: float = 1.0, copy_out: bool = False,
                    y_scale: Optional[torch.Tensor] = None, w_add: float = 0.0) -> Optional[torch.Tensor]:
    """In place on the fp32 residual ``[T, W]``: ``+= mult * rms_norm(y) * w_post`` (if ``y``; without ``w_post``:
    ``+= mult * y``; with ``y_scale`` ``[W]`` the addend is also scaled per channel), ``+= extra`` (if given); returns
    ``rms_norm(residual) * (w_add + w_pre)`` in ``out_dtype`` (``w_add = 1`` for weights stored as their distance from
    one; without ``w_pre``: the residual itself in ``out_dtype`` if ``copy_out``, else None).  One pass per row."""
    T, W = resid.shape
    if resid.is_cuda:
        out = torch.empty(T, W, dtype=out_dtype, device=resid.device) if (w_pre is not None or copy_out) else None
        code = _lib.dtype_code(out_dtype)
        if y_scale is not None and y_scale.dtype != out_dtype:
            raise ValueError("the channel scale is stored in the activation dtype")
        _lib.call("sxb_resid_norm_step", resid.data_ptr(), _lib.ptr(y), _lib.ptr(w_post), _lib.ptr(extra),
                  _lib.ptr(w_pre), _lib.ptr(out), T, W, float(eps), float(mult), code, _lib.ptr(y_scale), float(w_add),
                  _lib.stream_ptr())
        return out
    if y is not None:
        add = mult * (_rms(y.float(), eps) * w_post.float() if w_post is not None else y.float())
        resid += add * y_scale.float() if y_scale is not None else add
    if extra is not None:
        resid += extra
    if w_pre is None:
        return resid.to(out_dtype) if copy_out else None
    return (_rms(resid, eps) * (w_add + w_pre.float())).to(out_dtype)


# ------------------------------------------------------------------------------------------------ attention
def qk_norm_append(qkv: torch.Tensor, bias: Optional[torch.Tensor], kcache: torch.Tensor, vcache: torch.Tensor,
                   tok_seq: torch.Tensor, tok_pos: torch.Tensor, tables: torch.Tensor, Hq: int, G: int, d: int, dv: int,
                   eps: float, normalize: bool = True) -> torch.Tensor:
    """``qkv`` ``[T, Hq*d + G*d + G*dv]`` (+ ``bias``): q and k heads are divided by their root mean square (fp32), q is
    returned as fp32 ``[T, Hq, d]``, k and v are written to the paged caches ``[pages, block, G, d]`` /
    ``[pages, block, G, dv]`` at every token's (sequence, position)."""
    T = qkv.shape[0]
    bs = kcache.shape[1]
    if qkv.is_cuda:
        q = torch.empty(T, Hq, d, dtype=torch.float32, device=qkv.device)
        _lib.call("sxb_qk_norm_append", _rows(qkv).data_ptr(), qkv.stride(0), _lib.ptr(bias), q.data_ptr(),
                  kcache.data_ptr(), vcache.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(), tables.data_ptr(), T,
                  tables.shape[1], bs, Hq, G, d, dv, float(eps), int(normalize), _dt(qkv), _lib.stream_ptr())
        return q
    x = qkv[:, : (Hq + G) * d + G * dv].float() + (bias.float() if bias is not None else 0.0)
    q = x[:, : Hq * d].reshape(T, Hq, d)
    k = x[:, Hq * d: (Hq + G) * d].reshape(T, G, d)
    v = x[:, (Hq + G) * d:].reshape(T, G, dv)
    if normalize:
        q, k = _rms(q, eps), _rms(k, eps)
    page = tables[tok_seq.long(), (tok_pos // bs).long()].long()
    off = (tok_pos % bs).long()
    kcache[page, off] = k.to(kcache.dtype)
    vcache[page, off] = v.to(vcache.dtype)
    return q.contiguous()


def qkv_filter_norm_append(qkv: torch.Tensor, conv_w: Optional[torch.Tensor], state: Optional[torch.Tensor],
                           seq_info: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                           kcache: torch.Tensor, vcache: torch.Tensor, tok_seq: torch.Tensor, tok_pos: torch.Tensor,
                           tables: torch.Tensor, Hq: int, G: int, d: int, dv: int, eps: float, normalize: bool = True,
                           temp_coef: float = 0.0, temp_every: int = 1) -> torch.Tensor:
    """:func:`qk_norm_append` for projections ``qkv`` ``[T, >= Hq*d + G*d + G*dv]`` that first pass a short causal filter
    over time on every channel (``conv_w`` ``[C, taps]``, last column = current token; inputs before this batch's rows
    from ``state`` ``[slots, taps-1, C]``, before the sequence's start zero; None: no filter -- call
    :func:`conv_state_update` on the same columns afterwards).  q and k heads are then divided by their root mean square
    (``normalize``) and multiplied by ``q_w`` / ``k_w`` (``[d]``, shared by the heads; None: no weight); q also by
    ``1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)``.  Returns q fp32 ``[T, Hq, d]``; k, v go to the caches."""
    T = qkv.shape[0]
    bs = kcache.shape[1]
    C = (Hq + G) * d + G * dv
    taps = conv_w.shape[1] if conv_w is not None else 1
    if qkv.is_cuda:
        q = torch.empty(T, Hq, d, dtype=torch.float32, device=qkv.device)
        _lib.call("sxb_qkv_filter_norm_append", _rows(qkv).data_ptr(), qkv.stride(0), _lib.ptr(conv_w),
                  _lib.ptr(state if taps > 1 else None), seq_info.data_ptr(), _lib.ptr(q_w), _lib.ptr(k_w),
                  q.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(),
                  tables.data_ptr(), T, tables.shape[1], bs, Hq, G, d, dv, taps, float(eps), int(normalize),
                  float(temp_coef), int(temp_every), _dt(qkv), _lib.stream_ptr())
        return q
    x = qkv[:, :C].float()
    if conv_w is not None:
        wf = conv_w.float()
        y = torch.empty_like(x)
        for first, n, seen, slot in seq_info.tolist():
            hist = state[slot].float() if (seen > 0 and taps > 1) else torch.zeros(taps - 1, C)
            if 0 < seen < taps - 1:
                hist = hist.clone()
                hist[: taps - 1 - seen] = 0
            full = torch.cat([hist, x[first: first + n]], dim=0)
            acc = torch.zeros(n, C)
            for j in range(taps):
                acc += wf[:, j] * full[j: j + n]
            y[first: first + n] = acc
        x = y
    q = x[:, : Hq * d].reshape(T, Hq, d)
    k = x[:, Hq * d: (Hq + G) * d].reshape(T, G, d)
    v = x[:, (Hq + G) * d:].reshape(T, G, dv)
    if normalize:
        q, k = _rms(q, eps), _rms(k, eps)
    if q_w is not None:
        q = q * q_w.float()
    if k_w is not None:
        k = k * k_w.float()
    if temp_coef != 0.0:
        steps = torch.div(tok_pos.long() + 1, int(temp_every), rounding_mode="floor") + 1
        q = q * (1.0 + temp_coef * torch.log(steps.float()))[:, None, None]
    page = tables[tok_seq.long(), (tok_pos // bs).long()].long()
    off = (tok_pos % bs).long()
    kcache[page, off] = k.to(kcache.dtype)
    vcache[page, off] = v.to(vcache.dtype)
    return q.contiguous()


SHORT_ATOM = 16          # atoms of at most this many queries run one warp per (query, head)


def tiles_supported(d: int, dv: int) -> bool:
    return d % 4 == 0 and dv % 4 == 0 and d <= 256 and dv <= 256


def sink_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, sink: Optional[torch.Tensor],
                   tok_seq: torch.Tensor, tok_pos: torch.Tensor, tables: torch.Tensor, scale: float, chunk: int,
                   out_dtype: torch.dtype, atoms: Optional[torch.Tensor] = None, n_long: int = 0, window: int = 0,
                   value_cols: int = 0, value_col0: int = 0, dist_bias: Optional[torch.Tensor] = None,
                   gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Softmax attention of each token (fp32 ``q`` ``[T, Hq, d]``) over the cached keys ``lo..pos`` of its sequence,
    ``lo`` = first position of the token's chunk of ``chunk`` positions, or ``pos - window + 1`` (not below 0) for a
    sliding ``window``, or 0 (both 0: plain causal).  ``sink`` (fp32 ``[Hq]``) adds ``exp(sink[h])`` to the
    denominator.  Returns ``[T, Hq * dv]``.

    ``value_cols = dv > 0``: the values are the ``dv`` columns of the key rows that start at ``value_col0`` (one key
    head; ``vcache`` is not read) -- attention in a latent space where a key is ``[latent | extra]`` and its value the
    latent itself.

    ``dist_bias`` (fp32 ``[Hq, L]``): ``dist_bias[h, min(pos - j, L - 1)]`` is added to the scaled score of key ``j``.
    ``gate`` (``[T, Hq * dv]``, a column slice is fine): the result is multiplied by ``sigmoid(gate)``.

    With the batch's attention ``atoms`` (longest first) of which the first ``n_long`` hold more than
    :data:`SHORT_ATOM` queries, those run the tiled kernel (64 queries per CTA, K/V tiles shared by them) and the rest
    one warp per (query, head); without atoms every token takes the latter."""
    T, Hq, d = q.shape
    bs, G = kcache.shape[1], kcache.shape[2]
    if value_cols > 0:
        if G != 1:
            raise ValueError("values taken from the key rows need a single key head")
        dv, vsrc, v_pitch = int(value_cols), kcache, d
    else:
        dv, vsrc, v_pitch = vcache.shape[3], vcache, 0
    if q.is_cuda:
        if kcache.dtype != out_dtype or vsrc.dtype != out_dtype:
            raise ValueError("the caches and the output share one activation dtype")
        out = torch.empty(T, Hq * dv, dtype=out_dtype, device=q.device)
        vptr = vsrc.data_ptr() + (value_col0 * vsrc.element_size() if value_cols > 0 else 0)
        if value_cols > 0 and value_col0 % 8:
            raise ValueError("value columns start at a multiple of 8")
        if dist_bias is not None and (dist_bias.dtype != torch.float32 or not dist_bias.is_contiguous()
                                      or dist_bias.shape[0] != Hq):
            raise ValueError("the distance bias is a contiguous fp32 [heads, distances] table")
        if gate is not None and gate.dtype != out_dtype:
            raise ValueError("the gate has the activation dtype")
        extra = (_lib.ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[1],
                 None if gate is None else _rows(gate).data_ptr(), 0 if gate is None else gate.stride(0))
        if atoms is not None and n_long > 0 and tiles_supported(d, dv):
            _lib.call("sxb_sink_attention_atoms", q.data_ptr(), kcache.data_ptr(), vptr, _lib.ptr(sink),
                      out.data_ptr(), atoms.data_ptr(), atoms.shape[0], int(n_long), tables.data_ptr(), tables.shape[1],
                      bs, Hq, G, d, dv, float(scale), int(chunk), int(window), 0, v_pitch, *extra,
                      _lib.dtype_code(out_dtype), _lib.stream_ptr())
            return out
        _lib.call("sxb_sink_attention", q.data_ptr(), kcache.data_ptr(), vptr, _lib.ptr(sink),
                  out.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(), tables.data_ptr(), T, tables.shape[1], bs, Hq,
                  G, d, dv, float(scale), int(chunk), int(window), 0, v_pitch, *extra, _lib.dtype_code(out_dtype),
                  _lib.stream_ptr())
        return out
    out = torch.empty(T, Hq, dv, dtype=torch.float32)
    rep = Hq // G
    for t in range(T):
        pos = int(tok_pos[t])
        lo = (pos // chunk) * chunk if chunk > 0 else (max(0, pos - window + 1) if window > 0 else 0)
        js = torch.arange(lo, pos + 1)
        page = tables[int(tok_seq[t]), (js // bs)].long()
        k = kcache[page, js % bs].float().repeat_interleave(rep, dim=1)      # [n, Hq, d]
        if value_cols > 0:
            v = k[:, :, value_col0: value_col0 + dv]
        else:
            v = vcache[page, js % bs].float().repeat_interleave(rep, dim=1)
        s = torch.einsum("hd,nhd->hn", q[t], k) * scale
        if dist_bias is not None:
            s = s + dist_bias[:, (pos - js).clamp(max=dist_bias.shape[1] - 1)]
        if sink is not None:
            s = torch.cat([s, sink.float()[:, None]], dim=1)
        p = torch.softmax(s, dim=-1)[:, : js.numel()]
        out[t] = torch.einsum("hn,nhd->hd", p, v)
    out = out.reshape(T, Hq * dv)
    if gate is not None:
        out = out * torch.sigmoid(gate.float())
    return out.to(out_dtype)


# ------------------------------------------------------------------------------------------------ short convolution
def conv_silu(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
              seq_info: torch.Tensor, tok_seq: torch.Tensor) -> torch.Tensor:
    """Short causal per-channel filter + SiLU over the rows ``x`` ``[T, C]`` of a ragged batch; ``w`` ``[C, taps]`` (last
    column multiplies the current token), inputs before this batch's rows come from ``state`` ``[slots, taps-1, C]``,
    inputs before a sequence's start are zero.  Returns fp32 ``[T, C]``; call :func:`conv_state_update` afterwards."""
    T, C = x.shape
    taps = w.shape[1]
    if x.is_cuda:
        out = torch.empty(T, C, dtype=torch.float32, device=x.device)
        _lib.call("sxb_conv_silu", _rows(x).data_ptr(), x.stride(0), w.data_ptr(), _lib.ptr(bias), state.data_ptr(),
                  seq_info.data_ptr(), tok_seq.data_ptr(), out.data_ptr(), T, C, taps, _dt(x), _lib.stream_ptr())
        return out
    out = torch.empty(T, C, dtype=torch.float32)
    wf = w.float()
    for first, n, seen, slot in seq_info.tolist():
        hist = state[slot].float() if seen > 0 else torch.zeros(taps - 1, C)
        if 0 < seen < taps - 1:
            hist = hist.clone()
            hist[: taps - 1 - seen] = 0
        full = torch.cat([hist, x[first: first + n].float()], dim=0)
        acc = torch.zeros(n, C)
        for j in range(taps):
            acc += wf[:, taps - 1 - j] * full[taps - 1 - j: taps - 1 - j + n]
        if bias is not None:
            acc += bias.float()
        out[first: first + n] = torch.nn.functional.silu(acc)
    return out


def conv_state_update(x: torch.Tensor, state: torch.Tensor, seq_info: torch.Tensor) -> None:
    """Every sequence's slot of ``state`` ``[slots, taps-1, C]`` becomes the last ``taps-1`` rows of (its carried inputs
    followed by this batch's rows of ``x``)."""
    keep = state.shape[1]
    if keep == 0:
        return
    C = x.shape[1]
    if x.is_cuda:
        _lib.call("sxb_conv_state_update", _rows(x).data_ptr(), x.stride(0), state.data_ptr(), seq_info.data_ptr(),
                  seq_info.shape[0], C, keep + 1, _dt(x), _lib.stream_ptr())
        return
    for first, n, seen, slot in seq_info.tolist():
        hist = state[slot] if seen > 0 else torch.zeros_like(state[slot])
        if 0 < seen < keep:
            hist = hist.clone()
            hist[: keep - seen] = 0
        state[slot] = torch.cat([hist, x[first: first + n].to(state.dtype)], dim=0)[-keep:]


def unit_norm_heads(x: torch.Tensor, col0: int, n_heads: int, dim: int, mult: float, eps: float) -> None:
    """In place on fp32 rows: each head ``x[:, col0 + h*dim : col0 + (h+1)*dim]`` becomes ``x * mult / sqrt(sum x^2 + eps)``."""
    T = x.shape[0]
    if x.is_cuda:
        _lib.call("sxb_unit_norm_heads", _rows(x).data_ptr(), x.stride(0), col0, n_heads, dim, float(mult), float(eps), T,
                  _lib.stream_ptr())
        return
    v = x[:, col0: col0 + n_heads * dim].reshape(T, n_heads, dim)
    x[:, col0: col0 + n_heads * dim] = (v * mult / torch.sqrt(v.pow(2).sum(-1, keepdim=True) + eps)).reshape(T, -1)


def recurrence_gates(a_raw: torch.Tensor, b_raw: Optional[torch.Tensor], A_log: torch.Tensor, dt_bias: torch.Tensor,
                     mode: str):
    """fp32 ``(decay, beta)`` ``[T, H]`` of a linear recurrence from raw projections ``[T, H]`` (column slices allowed).
    ``"delta"``: ``beta = sigmoid(b_raw)``, ``decay = exp(-exp(A_log) * softplus(a_raw + dt_bias))``.
    ``"ssd"``: ``dt = softplus(a_raw + dt_bias)``, ``beta = dt``, ``decay = exp(-exp(A_log) * dt)``."""
    T, H = a_raw.shape
    if a_raw.is_cuda:
        decay = torch.empty(T, H, dtype=torch.float32, device=a_raw.device)
        beta = torch.empty_like(decay)
        b = a_raw if b_raw is None else b_raw
        if b.stride(0) != a_raw.stride(0):
            raise ValueError("a_raw and b_raw must share their row pitch")
        _lib.call("sxb_recurrence_gates", _rows(a_raw).data_ptr(), _rows(b).data_ptr(), a_raw.stride(0),
                  A_log.data_ptr(), dt_bias.data_ptr(), decay.data_ptr(), beta.data_ptr(), H, T,
                  0 if mode == "delta" else 1, _dt(a_raw), _lib.stream_ptr())
        return decay, beta
    dt = torch.nn.functional.softplus(a_raw.float() + dt_bias.float(), threshold=30.0)
    decay = torch.exp(-torch.exp(A_log.float()) * dt)
    beta = torch.sigmoid(b_raw.float()) if mode == "delta" else dt
    return decay, beta


def channel_decay_gates(a_raw: torch.Tensor, b_raw: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor,
                        H: int, n: int):
    """fp32 ``(decay [T, H*n], beta [T, H])`` of a delta rule whose decay differs per key channel: ``decay[t, h, c] =
    exp(-exp(A_log[h]) * softplus(a_raw[t, h*n + c] + dt_bias[h*n + c]))``, ``beta = sigmoid(b_raw)``.  ``a_raw``
    ``[T, H*n]`` and ``b_raw`` ``[T, H]`` may be column slices; ``A_log`` fp32 ``[H]``, ``dt_bias`` fp32 ``[H*n]``."""
    T = a_raw.shape[0]
    if a_raw.is_cuda:
        decay = torch.empty(T, H * n, dtype=torch.float32, device=a_raw.device)
        beta = torch.empty(T, H, dtype=torch.float32, device=a_raw.device)
        if b_raw.dtype != a_raw.dtype:
            raise ValueError("a_raw and b_raw share their dtype")
        _lib.call("sxb_channel_decay_gates", _rows(a_raw).data_ptr(), a_raw.stride(0), _rows(b_raw).data_ptr(),
                  b_raw.stride(0), A_log.data_ptr(), dt_bias.data_ptr(), decay.data_ptr(), beta.data_ptr(), T, H, n,
                  _dt(a_raw), _lib.stream_ptr())
        return decay, beta
    dt = torch.nn.functional.softplus(a_raw.float() + dt_bias.float(), threshold=30.0)
    decay = torch.exp(-torch.exp(A_log.float()).repeat_interleave(n)[None, :] * dt)
    return decay, torch.sigmoid(b_raw.float())


def linear_recurrence(kvec: torch.Tensor, qvec: torch.Tensor, val: torch.Tensor, decay: torch.Tensor,
                      beta: torch.Tensor, skip: Optional[torch.Tensor], state: torch.Tensor, seq_info: torch.Tensor,
                      H: int, G: int, n: int, dv: int, delta: bool) -> torch.Tensor:
    """Per sequence and head, rows in order: ``S <- decay S``; ``u = beta (v - S^T k)`` (``delta``) or ``beta v``;
    ``S <- S + k u^T``; ``o = S^T q (+ skip[h] v)``.  ``kvec`` / ``qvec`` fp32 ``[T, G*n]`` and ``val`` fp32
    ``[T, H*dv]`` may be column slices (``kvec`` and ``qvec`` with one row pitch); ``state`` fp32 ``[slots, H, dv, n]`` is
    read (zero for a sequence that has seen no token) and written back.  ``decay`` fp32 ``[T, H]`` is one factor per
    head; ``[T, H*n]`` one per head and key channel (it multiplies the state's entries of that channel).  Returns fp32
    ``[T, H*dv]``."""
    T = val.shape[0]
    per_channel = decay.shape[1] == H * n and n > 1
    if val.is_cuda:
        if kvec.stride(0) != qvec.stride(0):
            raise ValueError("kvec and qvec must share their row pitch")
        if not decay.is_contiguous() or decay.shape[1] not in (H, H * n):
            raise ValueError("decay is a contiguous [T, H] or [T, H*n] tensor")
        out = torch.empty(T, H * dv, dtype=torch.float32, device=val.device)
        _lib.call("sxb_linear_recurrence", _rows(kvec).data_ptr(), _rows(qvec).data_ptr(), kvec.stride(0),
                  _rows(val).data_ptr(), val.stride(0), decay.data_ptr(), beta.data_ptr(), _lib.ptr(skip),
                  state.data_ptr(), out.data_ptr(), seq_info.data_ptr(), seq_info.shape[0], H, G, n, dv, int(delta),
                  int(per_channel), _lib.stream_ptr())
        return out
    out = torch.empty(T, H, dv, dtype=torch.float32)
    rep = H // G
    for first, rows, seen, slot in seq_info.tolist():
        S = state[slot].clone() if seen > 0 else torch.zeros_like(state[slot])           # [H, dv, n]
        for t in range(first, first + rows):
            k = kvec[t].reshape(G, n).repeat_interleave(rep, dim=0)                      # [H, n]
            q = qvec[t].reshape(G, n).repeat_interleave(rep, dim=0)
            v = val[t].reshape(H, dv)
            S = S * (decay[t].reshape(H, 1, n) if per_channel else decay[t][:, None, None])
            u = beta[t][:, None] * ((v - torch.einsum("hvn,hn->hv", S, k)) if delta else v)
            S = S + u[:, :, None] * k[:, None, :]
            o = torch.einsum("hvn,hn->hv", S, q)
            if skip is not None:
                o = o + skip.float()[:, None] * v
            out[t] = o
        state[slot] = S
    return out.reshape(T, H * dv)


def group_norm_gate(y: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, group_size: int, eps: float,
                    gate_first: bool, out_dtype: torch.dtype, sigmoid: bool = False) -> torch.Tensor:
    """RMS norm over groups of ``group_size`` channels of fp32 ``y`` ``[T, C]`` with a SiLU gate ``[T, C]`` (column slice
    allowed) and a weight that repeats along the row.  ``gate_first``: ``norm(y * silu(gate)) * w``; else
    ``norm(y) * w * silu(gate)``.  ``sigmoid``: the gate is ``sigmoid(gate)`` instead of ``silu(gate)``."""
    T, C = y.shape
    if y.is_cuda:
        out = torch.empty(T, C, dtype=out_dtype, device=y.device)
        _lib.call("sxb_group_norm_gate", y.data_ptr(), _rows(gate).data_ptr(), gate.stride(0), w.data_ptr(), w.numel(),
                  out.data_ptr(), T, C, group_size, float(eps), int(gate_first) | (2 if sigmoid else 0),
                  _lib.dtype_code(out_dtype), _lib.stream_ptr())
        return out
    sg = torch.sigmoid(gate.float()) if sigmoid else torch.nn.functional.silu(gate.float())
    wf = w.float().repeat(C // w.numel())
    z = y * sg if gate_first else y
    z = _rms(z.reshape(T, C // group_size, group_size), eps).reshape(T, C) * wf
    return (z if gate_first else z * sg).to(out_dtype)


def gated_act_rows(x: torch.Tensor, act: str = "gelu", limit: float = 0.0) -> torch.Tensor:
    """``act(x[:, :F]) * x[:, F:]`` for rows of any width, bf16 or fp32 (``gelu`` is the tanh form).  ``clamped_swish``:
    ``a = min(x[:, :F], L)``, ``b = max(-L, min(x[:, F:], L))`` with ``L = limit``, result ``a * sigmoid(1.702 a) * (1 + b)``."""
    T, F2 = x.shape
    Fh = F2 // 2
    if x.is_cuda:
        x = x.contiguous()
        out = torch.empty(T, Fh, dtype=x.dtype, device=x.device)
        _lib.call("sxb_gated_act_rows", x.data_ptr(), out.data_ptr(), T, Fh, _ACTS[act], _dt(x), float(limit),
                  _lib.stream_ptr())
        return out
    g, u = x[:, :Fh].float(), x[:, Fh:].float()
    if act == "clamped_swish":
        g, u = g.clamp(max=limit), u.clamp(min=-limit, max=limit)
        return (g * torch.sigmoid(1.702 * g) * (u + 1.0)).to(x.dtype)
    a = {"gelu": lambda t: torch.nn.functional.gelu(t, approximate="tanh"), "silu": torch.nn.functional.silu,
         "relu": torch.relu, "identity": lambda t: t}[act](g)
    return (a * u).to(x.dtype)


def bias_act_rows(x: torch.Tensor, bias: Optional[torch.Tensor], act: str) -> torch.Tensor:
    """``act(x + bias)`` for rows of any width, bf16 or fp32; ``relu_sq`` is ``relu(z) ** 2``."""
    T, Fw = x.shape
    if x.is_cuda:
        x = x.contiguous()
        out = torch.empty_like(x)
        _lib.call("sxb_bias_act_rows", x.data_ptr(), _lib.ptr(bias), out.data_ptr(), T, Fw, _ACTS[act], _dt(x),
                  _lib.stream_ptr())
        return out
    z = x.float() + (bias.float() if bias is not None else 0.0)
    a = {"gelu": lambda t: torch.nn.functional.gelu(t, approximate="tanh"), "silu": torch.nn.functional.silu,
         "relu": torch.relu, "identity": lambda t: t, "relu_sq": lambda t: torch.relu(t) ** 2}[act](z)
    return a.to(x.dtype)


def power_norm_act(x: torch.Tensor, bias: Optional[torch.Tensor], coef: torch.Tensor, eps: float) -> torch.Tensor:
    """Three-power normalised activation of every row: ``z = x + bias``; ``p1 z / rms(z) + p2 z^2 / rms(z^2) + p3 z^3 /
    rms(z^3) + p0`` with ``(p1, p2, p3, p0) = coef`` (fp32 ``[4]``) and ``rms(u) = sqrt(mean(u^2) + eps)`` over the row; the
    sums are 32-bit, input and output share their dtype (bf16 or fp32)."""
    T, Fw = x.shape
    if x.is_cuda:
        x = x.contiguous()
        out = torch.empty_like(x)
        if coef.dtype != torch.float32 or coef.numel() != 4:
            raise ValueError("coef is an fp32 tensor of four numbers")
        _lib.call("sxb_power_norm_act", x.data_ptr(), _lib.ptr(bias), coef.data_ptr(), out.data_ptr(), T, Fw, float(eps),
                  _dt(x), _lib.stream_ptr())
        return out
    z = x.float() + (bias.float() if bias is not None else 0.0)
    c = coef.float()
    return (c[0] * _rms(z, eps) + c[1] * _rms(z * z, eps) + c[2] * _rms(z * z * z, eps) + c[3]).to(x.dtype)


def sigmoid_gate_rows_(x: torch.Tensor, gate: torch.Tensor, group: int = 1) -> torch.Tensor:
    """In place: ``x[t, c] *= sigmoid(gate[t, c // group])``; ``gate`` ``[T, W / group]`` (a column slice is fine) has one
    entry per channel (``group = 1``) or per run of ``group`` channels (a head)."""
    T, W = x.shape
    if x.is_cuda:
        if not x.is_contiguous() or gate.dtype != x.dtype:
            raise ValueError("expected contiguous rows and a gate of the same dtype")
        _lib.call("sxb_sigmoid_gate_rows", x.data_ptr(), _rows(gate).data_ptr(), gate.stride(0), T, W, int(group),
                  _dt(x), _lib.stream_ptr())
        return x
    g = torch.sigmoid(gate[:, : W // group].float()).repeat_interleave(group, dim=1)
    x.copy_((x.float() * g).to(x.dtype))
    return x


# ------------------------------------------------------------------------------------------------ post-norm layers
def conv_residual(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, seq_info: torch.Tensor, tok_seq: torch.Tensor,
                  out_dtype: torch.dtype) -> torch.Tensor:
    """``x + filter(x)`` over the fp32 rows ``x`` ``[T, C]`` of a ragged batch: ``filter(x)[t] = sum_j w[:, j] x[t - taps +
    1 + j]`` per channel (``w`` ``[C, taps]``), earlier rows of a sequence from ``state`` fp32 ``[slots, taps-1, C]``,
    rows before its start zero.  Returns ``out_dtype`` ``[T, C]``; call :func:`conv_state_update` on ``x`` afterwards."""
    T, C = x.shape
    taps = w.shape[1]
    if x.is_cuda:
        out = torch.empty(T, C, dtype=out_dtype, device=x.device)
        if w.dtype != out_dtype:
            raise ValueError("the filter is stored in the activation dtype")
        _lib.call("sxb_conv_residual", x.data_ptr(), w.data_ptr(), state.data_ptr(), seq_info.data_ptr(),
                  tok_seq.data_ptr(), out.data_ptr(), T, C, taps, _lib.dtype_code(out_dtype), _lib.stream_ptr())
        return out
    out = torch.empty(T, C, dtype=torch.float32)
    wf = w.float()
    for first, n, seen, slot in seq_info.tolist():
        hist = state[slot].float() if seen > 0 else torch.zeros(taps - 1, C)
        if 0 < seen < taps - 1:
            hist = hist.clone()
            hist[: taps - 1 - seen] = 0
        full = torch.cat([hist, x[first: first + n]], dim=0)
        acc = torch.zeros(n, C)
        for j in range(taps):
            acc += wf[:, j] * full[j: j + n]
        out[first: first + n] = x[first: first + n] + acc
    return out.to(out_dtype)


def post_norm_mix(x_in: torch.Tensor, y: torch.Tensor, gain: torch.Tensor, ls: torch.Tensor, x_out: torch.Tensor,
                  eps: float, stack: Optional[torch.Tensor] = None, n_prev: int = 0,
                  mixw: Optional[torch.Tensor] = None, mix_out: Optional[torch.Tensor] = None) -> None:
    """``x_out = x_in + ls * (y / rms(y) * gain)`` on fp32 rows (``gain`` fp32 ``[1]``, ``ls`` fp32 ``[W]``; ``x_out`` may
    be ``x_in``).  With ``mix_out``: ``mix_out = sum_{j < n_prev} mixw[j] * stack[j] + mixw[n_prev] * x_out`` (``stack``
    fp32 ``[>= n_prev, T, W]``, ``mixw`` fp32)."""
    T, W = x_in.shape
    if x_in.is_cuda:
        stride = stack.stride(0) if stack is not None else 0
        _lib.call("sxb_post_norm_mix", x_in.data_ptr(), y.data_ptr(), gain.data_ptr(), ls.data_ptr(), x_out.data_ptr(),
                  _lib.ptr(stack), stride, int(n_prev), _lib.ptr(mixw), _lib.ptr(mix_out), T, W, float(eps), _dt(y),
                  _lib.stream_ptr())
        return
    v = x_in + _rms(y.float(), eps) * gain.float() * ls.float()
    x_out.copy_(v)
    if mix_out is not None:
        m = torch.zeros_like(v)
        for j in range(n_prev):
            m += mixw[j] * stack[j]
        mix_out.copy_(m + mixw[n_prev] * v)


def rms_scale_rows(x: torch.Tensor, rows: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                   out_dtype: torch.dtype) -> torch.Tensor:
    """``x[rows] / rms * gain`` (one fp32 gain for all channels) of fp32 rows, in ``out_dtype``."""
    n = x.shape[0] if rows is None else rows.numel()
    W = x.shape[1]
    if x.is_cuda:
        out = torch.empty(n, W, dtype=out_dtype, device=x.device)
        _lib.call("sxb_rms_scale_rows", x.data_ptr(), _lib.ptr(rows), gain.data_ptr(), out.data_ptr(), n, W, float(eps),
                  _lib.dtype_code(out_dtype), _lib.stream_ptr())
        return out
    sel = x if rows is None else x.index_select(0, rows.long())
    return (_rms(sel, eps) * gain.float()).to(out_dtype)


def rms_norm_slice(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm with weight over the columns of ``x`` (a column slice of a wider matrix is fine), computed in fp32."""
    T, n = x.shape
    if x.is_cuda:
        out = torch.empty(T, n, dtype=x.dtype, device=x.device)
        _lib.call("sxb_rms_norm_slice", _rows(x).data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), T, n, float(eps),
                  _dt(x), _lib.stream_ptr())
        return out
    return (_rms(x.float(), eps) * w.float()).to(x.dtype)


# ------------------------------------------------------------------------------------------------ latent attention
def _rope_pairs(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, amp: float = 1.0) -> torch.Tensor:
    """Rotate the pairs (2i, 2i+1), i < len(inv_freq), of the last axis of fp32 ``x`` ``[T, ..., n]`` by ``pos * inv_freq``
    (cos and sin times ``amp``)."""
    nd = 2 * inv_freq.numel()
    ang = pos.float()[:, None] * inv_freq.float()[None, :]
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (nd // 2,)
    cs, sn = (ang.cos() * amp).view(shape), (ang.sin() * amp).view(shape)
    out = x.clone()
    u, v = x[..., 0:nd:2], x[..., 1:nd:2]
    out[..., 0:nd:2] = u * cs - v * sn
    out[..., 1:nd:2] = v * cs + u * sn
    return out


def latent_qk_prepare(q: torch.Tensor, q_abs: torch.Tensor, kv: torch.Tensor, w_norm: torch.Tensor,
                      inv_freq: torch.Tensor, cache: torch.Tensor, tok_seq: torch.Tensor, tok_pos: torch.Tensor,
                      tables: torch.Tensor, H: int, dim: int, rot: int, eps: float, amp: float = 1.0) -> torch.Tensor:
    """Latent attention, per token.  ``kv`` ``[T, r + rot]``: ``cache[page, offset, 0] = [kv[:r] / rms * w_norm |
    rope(kv[r:])]`` (``cache`` ``[pages, block, 1, r + rot]``).  ``q`` ``[T, H * (dim + rot)]`` (heads laid out
    ``[dim unrotated | rot rotated]``) and ``q_abs`` ``[T, H, r]`` (any strides with unit inner stride; the unrotated
    part of every query head carried through the key up-projection): returns fp32 ``[T, H, r + rot] = [q_abs |
    rope(q[..., dim:])]``.  ``rope`` turns the pairs ``(2i, 2i+1)``, ``i < len(inv_freq)``, by ``pos * inv_freq[i]`` and
    multiplies the turned channels by ``amp``."""
    T = q.shape[0]
    r = kv.shape[1] - rot
    bs = cache.shape[1]
    if q.is_cuda:
        out = torch.empty(T, H, r + rot, dtype=torch.float32, device=q.device)
        _lib.call("sxb_latent_qk_prepare", _rows(q).data_ptr(), q.stride(0), _rows(q_abs).data_ptr(), q_abs.stride(0),
                  q_abs.stride(1), _rows(kv).data_ptr(), kv.stride(0), w_norm.data_ptr(), inv_freq.data_ptr(),
                  out.data_ptr(), cache.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(), tables.data_ptr(), T,
                  tables.shape[1], bs, H, dim, rot, r, 2 * inv_freq.numel(), float(eps), _dt(q), float(amp),
                  _lib.stream_ptr())
        return out
    c = (_rms(kv[:, :r].float(), eps) * w_norm.float()).to(cache.dtype)
    kr = _rope_pairs(kv[:, r:].float(), tok_pos, inv_freq, amp).to(cache.dtype)
    page = tables[tok_seq.long(), (tok_pos // bs).long()].long()
    off = (tok_pos % bs).long()
    cache[page, off, 0] = torch.cat([c, kr], dim=1)
    qr = _rope_pairs(q.reshape(T, H, dim + rot)[:, :, dim:].float(), tok_pos, inv_freq, amp)
    return torch.cat([q_abs.float(), qr], dim=2).contiguous()


# ------------------------------------------------------------------------------------------------ matrix-memory LSTM
def mlstm_prepare(proj: torch.Tensor, H: int, n: int, dv: int, qscale: float) -> torch.Tensor:
    """fp32 ``[T, 2 H n + H (dv + 1)] = [q * qscale | k | per head (v, 1)]`` from projection rows that start with
    ``q (H n) | k (H n) | v (H dv)``; the constant channel makes the recurrence carry the normaliser ``sum decay.. k``."""
    T = proj.shape[0]
    if proj.is_cuda:
        buf = torch.empty(T, 2 * H * n + H * (dv + 1), dtype=torch.float32, device=proj.device)
        _lib.call("sxb_mlstm_prepare", _rows(proj).data_ptr(), proj.stride(0), buf.data_ptr(), T, H, n, dv, float(qscale),
                  _dt(proj), _lib.stream_ptr())
        return buf
    q = proj[:, : H * n].float() * qscale
    k = proj[:, H * n: 2 * H * n].float()
    v = proj[:, 2 * H * n: 2 * H * n + H * dv].float().reshape(T, H, dv)
    v1 = torch.cat([v, torch.ones(T, H, 1)], dim=2).reshape(T, H * (dv + 1))
    return torch.cat([q, k, v1], dim=1)


def mlstm_gate_scan(raw_i: torch.Tensor, raw_f: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float,
                    mstate: torch.Tensor, seq_info: torch.Tensor):
    """Exponential gating with a running maximum.  ``raw_i`` / ``raw_f`` ``[T, H]`` (column slices of one matrix),
    biases fp32 ``[H]``: ``i = cap tanh((raw_i + b_i) / cap)``, ``f = logsigmoid(cap tanh((raw_f + b_f) / cap))``,
    ``m_t = max(f_t + m_(t-1), i_t)`` with ``m`` from ``mstate`` fp32 ``[slots, H]`` (0 for a sequence that has seen no
    token; written back).  Returns fp32 ``[T, H]`` ``(decay = exp(f + m_(t-1) - m_t), beta = exp(i - m_t), m_t)``."""
    T, H = raw_i.shape
    if raw_i.is_cuda:
        if raw_i.stride(0) != raw_f.stride(0):
            raise ValueError("raw_i and raw_f must share their row pitch")
        decay = torch.empty(T, H, dtype=torch.float32, device=raw_i.device)
        beta, mt = torch.empty_like(decay), torch.empty_like(decay)
        _lib.call("sxb_mlstm_gate_scan", _rows(raw_i).data_ptr(), _rows(raw_f).data_ptr(), raw_i.stride(0),
                  bias_i.data_ptr(), bias_f.data_ptr(), float(cap), mstate.data_ptr(), decay.data_ptr(), beta.data_ptr(),
                  mt.data_ptr(), seq_info.data_ptr(), seq_info.shape[0], T, H, _dt(raw_i), _lib.stream_ptr())
        return decay, beta, mt
    ig = cap * torch.tanh((raw_i.float() + bias_i.float()) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((raw_f.float() + bias_f.float()) / cap))
    decay, beta, mt = torch.empty(T, H), torch.empty(T, H), torch.empty(T, H)
    for first, rows, seen, slot in seq_info.tolist():
        m = mstate[slot].clone() if seen > 0 else torch.zeros(H)
        for t in range(first, first + rows):
            mn = torch.maximum(fg[t] + m, ig[t])
            decay[t], beta[t], mt[t] = torch.exp(fg[t] + m - mn), torch.exp(ig[t] - mn), mn
            m = mn
        mstate[slot] = m
    return decay, beta, mt


def mlstm_output(o: torch.Tensor, mt: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, H: int, dv: int, eps: float,
                 out_dtype: torch.dtype) -> torch.Tensor:
    """``o`` fp32 ``[T, H (dv + 1)]`` (read-out of the values and, last per head, of the normaliser): per head
    ``h = o[:dv] / (max(|o[dv]|, exp(-m_t)) + 1e-6)``, then ``h / rms(h) * w * sigmoid(gate)`` in ``out_dtype``
    ``[T, H dv]``."""
    T = o.shape[0]
    if o.is_cuda:
        out = torch.empty(T, H * dv, dtype=out_dtype, device=o.device)
        _lib.call("sxb_mlstm_output", o.data_ptr(), mt.data_ptr(), _rows(gate).data_ptr(), gate.stride(0), w.data_ptr(),
                  out.data_ptr(), T, H, dv, float(eps), _lib.dtype_code(out_dtype), _lib.stream_ptr())
        return out
    oo = o.reshape(T, H, dv + 1)
    den = torch.maximum(oo[:, :, dv].abs(), torch.exp(-mt)) + 1e-6
    h = _rms(oo[:, :, :dv] / den[:, :, None], eps).reshape(T, H * dv)
    return (h * w.float() * torch.sigmoid(gate.float())).to(out_dtype)


# ------------------------------------------------------------------------------------------------ small row ops
def side_gate(gx: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, col0: int, dim: int, out_width: int) -> torch.Tensor:
    """``[T, out_width]``: ``gelu_tanh(gx[:, :dim]) * table[ids, col0 : col0 + dim]``, zero in the columns from ``dim``
    on (padding for the product that follows).  ``gx`` may be a column slice."""
    T = gx.shape[0]
    if gx.is_cuda:
        out = torch.empty(T, out_width, dtype=gx.dtype, device=gx.device)
        if table.dtype != gx.dtype:
            raise ValueError("the table is stored in the activation dtype")
        _lib.call("sxb_side_gate", _rows(gx).data_ptr(), gx.stride(0), _rows(table).data_ptr(), table.stride(0),
                  ids.data_ptr(), out.data_ptr(), T, int(dim), int(out_width), int(col0), _dt(gx), _lib.stream_ptr())
        return out
    g = torch.nn.functional.gelu(gx[:, :dim].float(), approximate="tanh") * table[ids.long(), col0: col0 + dim].float()
    out = torch.zeros(T, out_width, dtype=gx.dtype)
    out[:, :dim] = g.to(gx.dtype)
    return out


def scale_softcap_(x: torch.Tensor, scale: float, cap: float) -> torch.Tensor:
    """In place on fp32 ``x``: ``x * scale``, then ``cap * tanh(x / cap)`` when ``cap > 0``."""
    if x.is_cuda:
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise ValueError("expected a contiguous fp32 tensor")
        _lib.call("sxb_scale_softcap", x.data_ptr(), x.numel(), float(scale), float(cap), _lib.stream_ptr())
        return x
    x.mul_(scale)
    if cap > 0:
        x.copy_(cap * torch.tanh(x / cap))
    return x


def row_gate_add_(acc: torch.Tensor, y: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """In place: ``acc[t] += sigmoid(gate[t]) * y[t]``; ``gate`` fp32 ``[T]`` (any stride), ``acc`` / ``y`` ``[T, W]``."""
    T, W = acc.shape
    if acc.is_cuda:
        if gate.dtype != torch.float32 or not acc.is_contiguous() or not y.is_contiguous() or y.dtype != acc.dtype:
            raise ValueError("expected contiguous rows of one dtype and an fp32 gate")
        _lib.call("sxb_row_gate_add", acc.data_ptr(), y.data_ptr(), gate.data_ptr(), gate.stride(0), T, W, _dt(acc),
                  _lib.stream_ptr())
        return acc
    acc.copy_((acc.float() + torch.sigmoid(gate.float())[:, None] * y.float()).to(acc.dtype))
    return acc


ROUTER_ROWS = 16         # router rows the fused product takes


def router_logits(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 ``[T, R] = x w^T + bias`` with 32-bit products and sums: ``x`` ``[T, W]`` in the activation dtype (bf16 values
    enter as they are), ``w`` fp32 ``[R, W]``, ``bias`` fp32 ``[R]``.  The kernel takes up to :data:`ROUTER_ROWS` rows and
    widths that are multiples of 4; anything else is the library's fp32 product of the converted rows."""
    T, W = x.shape
    R = w.shape[0]
    if (x.is_cuda and R <= ROUTER_ROWS and W % 4 == 0 and w.dtype == torch.float32 and w.is_contiguous()
            and x.dtype in (torch.bfloat16, torch.float32) and x.stride(1) == 1
            and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0
            and (bias is None or bias.dtype == torch.float32)):
        out = torch.empty(T, R, dtype=torch.float32, device=x.device)
        _lib.call("sxb_router_logits", x.data_ptr(), x.stride(0), w.data_ptr(), _lib.ptr(bias), out.data_ptr(), T, W, R,
                  _dt(x), _lib.stream_ptr())
        return out
    return torch.nn.functional.linear(x.float(), w.float(), None if bias is None else bias.float())
