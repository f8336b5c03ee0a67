"""Plain float64 evaluation of a Pifazen stack, one function per mechanism, whole sequences at a time and nothing
cached.  It shares no code with the package: the tests compare the engine (paged cache, carried state, ragged batches,
kernels) with it.

``config`` is the model's ``config.json`` object and ``tensors`` maps checkpoint names to arrays (any float dtype).

The stack: ``x = embed[token]``; pre-norm layers ``x += ls1 * mixer(n1(x))``, ``x += ls2 * ff(n2(x))`` with
``n(x) = x / rms(x) * (1 + w)``; a layer may borrow another layer's tensors (``weights_of``); final norm of the same form
and the embedding table as the head.  Mixers: a gated delta rule whose decay differs per key channel, and two forms of
latent attention with an output gate.  Feed-forwards: a dense one with a three-power normalised activation, or clamped
gated experts chosen among groups, some of which are the identity.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the distance from one."""
    return rms_norm(x, None, eps) * (1.0 + w)


def causal_filter(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``u`` [T, C], ``w`` [C, taps]: ``y[t] = sum_j w[:, j] * u[t - taps + 1 + j]`` with zeros before the start."""
    T, _ = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ------------------------------------------------------------------------------------------------ rotation
def rotary_frequencies(rot: Dict) -> (List[float], float):
    """Angular frequency of every pair and the factor on cos and sin.  With ``rot["scaling"]`` the pairs whose wavelength
    exceeds the original context are slowed by ``factor``, those that turn fast keep their frequency, the ones between are
    blended along a linear ramp over the pair index, and the amplitude grows with the logarithm of the factor."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, freqs: List[float], amp: float) -> torch.Tensor:
    """``x`` [T, ..., n]: the pairs (2i, 2i+1), i < len(freqs), of the token at position p turn by ``p * freqs[i]``; the
    turned channels are multiplied by ``amp``; the channels behind them pass."""
    T = x.shape[0]
    out = x.clone()
    for p in range(T):
        for i, f in enumerate(freqs):
            a = p * f
            c, s = math.cos(a) * amp, math.sin(a) * amp
            u, v = x[p, ..., 2 * i], x[p, ..., 2 * i + 1]
            out[p, ..., 2 * i] = u * c - v * s
            out[p, ..., 2 * i + 1] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ mixers
def latent_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: Dict, eps: float, direct_query: bool) -> torch.Tensor:
    """Keys and values as up-projections of one normalised latent per token, a single rotated key slice that every head uses.
    ``direct_query``: queries straight from the input and one gate per head; else queries through a normalised latent
    and one gate per output channel."""
    T = h.shape[0]
    H, d, rd, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    freqs, amp = rotary_frequencies(m["rot"])
    if direct_query:
        q = h @ P["q"].T
    else:
        q = rms_norm(h @ P["dq"].T, P["dq.norm"], eps) @ P["uq"].T
    q = q.view(T, H, d + rd)
    q_plain, q_rot = q[:, :, :d], rotate_pairs(q[:, :, d:], freqs, amp)
    kv = h @ P["dkv"].T
    c = rms_norm(kv[:, :r], P["dkv.norm"], eps)
    k_rot = rotate_pairs(kv[:, r:], freqs, amp)                         # [T, rd], one for all heads
    k_plain = (c @ P["uk"].T).view(T, H, d)
    v = (c @ P["uv"].T).view(T, H, dv)
    scale = float(m["scale"])
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * scale
        s = s.masked_fill(~causal, float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, hd]
    gate = torch.sigmoid(h @ P["g"].T)
    if direct_query:
        out = out * gate[:, :, None]                                     # [T, H] one per head
    else:
        out = out * gate.view(T, H, dv)
    return out.reshape(T, H * dv) @ P["o"].T


def unit_vectors(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def channel_delta(h: torch.Tensor, P: Dict[str, torch.Tensor], m: Dict, eps: float,
                  state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gated delta rule with a separate decay for every key channel of every head.  Matrix memory ``S`` [key channel, value channel] per
    head: ``S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``."""
    T = h.shape[0]
    H, G, n, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(causal_filter(h @ P["q"].T, P["q.conv"])).view(T, G, n)
    k = silu(causal_filter(h @ P["k"].T, P["k.conv"])).view(T, G, n)
    v = silu(causal_filter(h @ P["v"].T, P["v.conv"])).view(T, H, dv)
    q = unit_vectors(q) * n ** -0.5
    k = unit_vectors(k)
    beta = torch.sigmoid(h @ P["b"].T)                                                  # [T, H]
    step = softplus((h @ P["a1"].T) @ P["a2"].T + P["dt_bias"]).view(T, H, n)
    g = torch.exp(-torch.exp(P["A_log"])[None, :, None] * step)                       # [T, H, n]
    rep = H // G
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(n, dv, dtype=F64) if state is None else state[hd]
        kh, qh = k[:, hd // rep], q[:, hd // rep]
        for t in range(T):
            S = g[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ kh[t])
            S = S + torch.outer(kh[t], u)
            out[t, hd] = S.T @ qh[t]
    gate = torch.sigmoid((h @ P["g1"].T) @ P["g2"].T).view(T, H, dv)
    out = rms_norm(out, P["norm"], eps) * gate
    return out.reshape(T, H * dv) @ P["o"].T


# ------------------------------------------------------------------------------------------------ feed-forwards
def three_power_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """``p1 R(z) + p2 R(z^2) + p3 R(z^3) + p0`` with ``R(u) = u / rms(u)`` over a row and ``coef = (p1, p2, p3, p0)``."""
    return (coef[0] * rms_norm(z, None, eps) + coef[1] * rms_norm(z * z, None, eps)
            + coef[2] * rms_norm(z * z * z, None, eps) + coef[3])


def dense_ff(h: torch.Tensor, P: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    z = h @ P["up"].T + P["up.b"]
    return three_power_norm(z, P["act"], eps) @ P["down"].T + P["down.b"]


def clamped_expert(h: torch.Tensor, gate_w, up_w, down_w, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate_w.T, max=limit)
    u = torch.clamp(h @ up_w.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down_w.T


def route(z: torch.Tensor, correction: torch.Tensor, top: int, n_groups: int, keep: int, scale: float):
    """``z`` [T, R] router outputs -> (chosen [T, top], weights [T, top]).  Choice by ``softmax(z) + correction`` inside
    the ``keep`` contiguous blocks whose best member scores highest; weights from the softmax alone."""
    T, R = z.shape
    s = torch.softmax(z, dim=-1)
    choice = s + correction
    per = R // n_groups
    best = choice.view(T, n_groups, per).max(dim=-1).values
    kept = torch.topk(best, keep, dim=-1).indices
    allowed = torch.zeros(T, n_groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), float("-inf"))
    chosen = torch.topk(masked, top, dim=-1).indices
    w = s.gather(1, chosen)
    w = w / (w.sum(dim=-1, keepdim=True) + 1e-20) * scale
    return chosen, w


def expert_ff(h: torch.Tensor, P: Dict[str, torch.Tensor], mlp: Dict) -> torch.Tensor:
    r = mlp["router"]
    n_real, n_id = int(r["experts"]), int(r.get("identity", 0))
    groups = r.get("groups") or {"count": 1, "keep": 1}
    z = h @ P["router"].T
    assert z.shape[1] == n_real + n_id
    chosen, w = route(z, P["correction"], int(r["top"]), int(groups["count"]), int(groups["keep"]),
                      float(r.get("scale", 1.0)))
    limit = float(mlp["expert"]["limit"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t].tolist(), w[t]):
            if e >= n_real:
                out[t] += wt * h[t]
            else:
                out[t] += wt * clamped_expert(h[t: t + 1], P[f"e{e}.gate"], P[f"e{e}.up"], P[f"e{e}.down"], limit)[0]
    return out


# ------------------------------------------------------------------------------------------------ the stack
def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def owner(config: Dict, i: int) -> int:
    """Index of the layer whose tensors layer ``i`` uses."""
    seen = set()
    while config["layers"][i].get("weights_of") is not None:
        assert i not in seen
        seen.add(i)
        i = int(config["layers"][i]["weights_of"])
    return i


def mixer(kind: str, h, P, m, eps):
    if kind == "channel_delta":
        return channel_delta(h, P, m, eps)
    if kind == "latent_attention":
        return latent_attention(h, P, m, eps, direct_query=False)
    if kind == "latent_attention_2":
        return latent_attention(h, P, m, eps, direct_query=True)
    raise ValueError(kind)


def forward(config: Dict, tensors: Dict[str, torch.Tensor], tokens: List[int], layer_outputs: Optional[list] = None
            ) -> torch.Tensor:
    """float64 logits ``[len(tokens), vocab]`` of one sequence; ``layer_outputs`` collects the stream behind every layer."""
    eps = float(config["norm"]["eps"])
    embed = tensors["embed"].to(F64)
    x = embed[torch.tensor(tokens, dtype=torch.long)]
    for i, L in enumerate(config["layers"]):
        p = f"l{owner(config, i)}."
        g = {k: tensors[p + k].to(F64) for k in ("norm1", "ls1")}
        x = x + g["ls1"] * mixer(L["type"], offset_norm(x, g["norm1"], eps), sub(tensors, p + "mix."), L["mixer"], eps)
        mlp = L.get("mlp")
        if mlp is not None:
            hin = offset_norm(x, tensors[p + "norm2"].to(F64), eps)
            P = sub(tensors, p + "mlp.")
            y = dense_ff(hin, P, eps) if mlp["kind"] == "dense" else expert_ff(hin, P, mlp)
            x = x + tensors[p + "ls2"].to(F64) * y
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return offset_norm(x, tensors["final.norm"].to(F64), eps) @ embed.T


# ------------------------------------------------------------------------------------------------ random checkpoints
def random_weights(config: Dict, seed: int = 0, dtype=torch.bfloat16, rank: int = 6) -> Dict[str, torch.Tensor]:
    """A checkpoint of the configuration's shapes; values are rounded to ``dtype`` so that both sides read the same.
    ``rank`` is the inner size of the delta rule's two-step projections (a tensor shape, not a configuration entry)."""
    gen = torch.Generator().manual_seed(seed)
    W = int(config["width"])

    def rnd(*shape, std=1.0):
        return (torch.randn(*shape, generator=gen) * std).to(dtype)

    def lin(o, i, gain=1.0):
        return rnd(o, i, std=gain / math.sqrt(i))

    t: Dict[str, torch.Tensor] = {"embed": rnd(int(config["vocab"]), W), "final.norm": rnd(W, std=0.2)}
    for i, L in enumerate(config["layers"]):
        if L.get("weights_of") is not None:
            continue
        p, m, kind = f"l{i}.", L["mixer"], L["type"]
        t[p + "norm1"], t[p + "ls1"] = rnd(W, std=0.2), (0.5 + 0.5 * torch.rand(W, generator=gen)).to(dtype)
        x = p + "mix."
        if kind == "channel_delta":
            H, G, n, dv, taps = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m["conv"])
            for name, rows in (("q", G * n), ("k", G * n), ("v", H * dv)):
                t[x + name] = lin(rows, W, 2.0)
                t[x + name + ".conv"] = rnd(rows, taps, std=0.6)
            t[x + "b"] = lin(H, W, 2.0)
            t[x + "A_log"] = (torch.rand(H, generator=gen) * 2.0 - 2.0).to(dtype)
            t[x + "a1"], t[x + "a2"] = lin(rank, W, 2.0), lin(H * n, rank, 2.0)
            t[x + "dt_bias"] = rnd(H * n, std=1.0)
            t[x + "g1"], t[x + "g2"] = lin(rank, W, 2.0), lin(H * dv, rank, 2.0)
            t[x + "norm"] = (1.0 + rnd(dv, std=0.2).float()).to(dtype)
            t[x + "o"] = lin(W, H * dv)
        else:
            H, d, rd, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
            if kind == "latent_attention":
                qr = int(m["q_rank"])
                t[x + "dq"], t[x + "dq.norm"] = lin(qr, W, 2.0), (1.0 + rnd(qr, std=0.2).float()).to(dtype)
                t[x + "uq"] = lin(H * (d + rd), qr, 2.0)
                t[x + "g"] = lin(H * dv, W, 2.0)
            else:
                t[x + "q"] = lin(H * (d + rd), W, 2.0)
                t[x + "g"] = lin(H, W, 2.0)
            t[x + "dkv"], t[x + "dkv.norm"] = lin(r + rd, W, 2.0), (1.0 + rnd(r, std=0.2).float()).to(dtype)
            t[x + "uk"], t[x + "uv"] = lin(H * d, r, 2.0), lin(H * dv, r)
            t[x + "o"] = lin(W, H * dv)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        t[p + "norm2"], t[p + "ls2"] = rnd(W, std=0.2), (0.5 + 0.5 * torch.rand(W, generator=gen)).to(dtype)
        f = p + "mlp."
        if mlp["kind"] == "dense":
            ff = int(mlp["ff"])
            t[f + "up"], t[f + "up.b"] = lin(ff, W), rnd(ff, std=0.3)
            t[f + "down"], t[f + "down.b"] = lin(W, ff), rnd(W, std=0.3)
            t[f + "act"] = torch.tensor([0.7, 0.4, 0.3, 0.1]).to(dtype)
        else:
            r_ = mlp["router"]
            n_real, n_id, ff = int(r_["experts"]), int(r_.get("identity", 0)), int(mlp["expert"]["ff"])
            for e in range(n_real):
                t[f"{f}e{e}.gate"], t[f"{f}e{e}.up"] = lin(ff, W, 1.5), lin(ff, W, 1.5)
                t[f"{f}e{e}.down"] = lin(W, ff)
            t[f + "router"] = lin(n_real + n_id, W, 3.0)
            t[f + "correction"] = rnd(n_real + n_id, std=0.1)
    return t
