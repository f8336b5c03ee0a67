"""Plain float64 evaluation of a Ridazen stack, one function per mechanism, whole sequences at a time and nothing
cached.  It shares no code with the package: the tests compare the engine (paged cache, carried filter inputs, ragged
batches, kernels) with it.

``config`` is the model's ``config.json`` object and ``tensors`` maps checkpoint names to arrays (any float dtype).

The stack: ``x = embed[token]``; layers ``x += m * mixer(norm1(x))``, ``x += m * ff(norm2(x))``, then a per-layer token
input ``x += m * rms(proj(gelu(gate x) * e_i[token])) * w``; a span of layers may run several times (each pass adds the
embedding output again before its first layer); final norm, head, scale, soft cap.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_filter(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``u`` [T, C], ``w`` [C, taps]: ``y[t] = sum_j w[:, j] * u[t - taps + 1 + j]`` with zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def distance_bucket(n: int, rows: int, far: int) -> int:
    """Row of the distance table for a distance ``n >= 0``: exact below half the rows, logarithmic up to ``far``."""
    half = rows // 2
    if n < half:
        return n
    r = math.log(n / half) / math.log(far / half) * (rows - half)
    return min(rows - 1, half + int(math.floor(r + 1e-9)))


def distance_bias_matrix(column: torch.Tensor, T: int, far: int) -> torch.Tensor:
    """[T, T]: entry (i, j) is the table entry of distance i - j for j <= i (0 above the diagonal)."""
    per_distance = torch.stack([column[distance_bucket(n, column.shape[0], far)] for n in range(T)])
    i = torch.arange(T)
    return per_distance[(i[:, None] - i[None, :]).clamp(min=0)]


def query_temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log(((p + 1) // every) + 1)


def attention_mixer(h: torch.Tensor, P: Dict[str, torch.Tensor], m: Dict, eps: float) -> torch.Tensor:
    """``h`` [T, W] -> [T, W]; ``P`` holds the mixer's tensors without their prefix (``q``, ``q.conv``, ``q.norm`` ...)."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q, k, v = h @ P["q"].T, h @ P["k"].T, h @ P["v"].T
    if "q.conv" in P:
        q, k, v = causal_filter(q, P["q.conv"]), causal_filter(k, P["k.conv"]), causal_filter(v, P["v.conv"])
    q = rms_norm(q.view(T, H, d), P["q.norm"], eps)
    k = rms_norm(k.view(T, G, d), P["k.norm"], eps)
    v = v.view(T, G, dv)
    qt = m.get("q_temp")
    if qt:
        temp = torch.tensor([query_temperature(p, float(qt["coef"]), int(qt["every"])) for p in range(T)], dtype=F64)
        q = q * temp[:, None, None]
    rel = P.get("rel")
    out = torch.zeros(T, H, dv, dtype=F64)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ k[:, g].T) * float(m["scale"])
        if rel is not None:
            s = s + distance_bias_matrix(rel[:, hq], T, int(m["bias_max"]))
        w = torch.softmax(s.masked_fill(~causal, float("-inf")), dim=-1)
        out[:, hq] = w @ v[:, g]
    ctx = out.reshape(T, H * dv) * torch.sigmoid(h @ P["g"].T)
    return ctx @ P["o"].T


def expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (torch.relu(h @ up.T) ** 2) @ down.T


def moe_ff(h: torch.Tensor, P: Dict[str, torch.Tensor], mlp: Dict) -> torch.Tensor:
    T = h.shape[0]
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ P["router"].T + P["router.b"]
    y = torch.zeros(T, P["e0.down"].shape[0], dtype=F64)
    for t in range(T):
        pick = torch.topk(z[t], top).indices
        wts = torch.softmax(z[t, pick], dim=0)
        for e, wt in zip(pick.tolist(), wts):
            y[t] += wt * expert(h[t: t + 1], P[f"e{e}.up"], P[f"e{e}.down"])[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ P["shared.sg"].T)           # [T, 1]
        y = y + gate * expert(h, P["shared.up"], P["shared.down"])
    return y


def token_side(x: torch.Tensor, tokens: List[int], table: torch.Tensor, P: Dict[str, torch.Tensor], layer: int,
               dim: int, m: float, eps: float) -> torch.Tensor:
    e = table[tokens][:, layer * dim: (layer + 1) * dim]
    g = gelu_tanh(x @ P["gate"].T) * e
    y = g @ P["proj"].T
    return x + m * rms_norm(y, P["norm"], eps)


def _sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def execution_order(config: Dict) -> List[Tuple[int, bool]]:
    n = len(config["layers"])
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for rep in range(times):
        order += [(i, rep > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(config: Dict, tensors: Dict[str, torch.Tensor], tokens: List[int], layer_outputs: Optional[list] = None
            ) -> torch.Tensor:
    """Logits [T, vocab] of one sequence."""
    eps, m = float(config["norm"]["eps"]), float(config["residual_mult"])
    side = config.get("token_side")
    x0 = tensors["embed"].to(F64)[tokens]
    x = x0.clone()
    for i, again in execution_order(config):
        L = config["layers"][i]
        p = f"l{i}."
        if again:
            x = x + x0
        if L["type"] != "attention":
            raise ValueError(L["type"])
        x = x + m * attention_mixer(rms_norm(x, tensors[p + "norm1"].to(F64), eps), _sub(tensors, p + "mix."),
                                    L["mixer"], eps)
        if L.get("mlp") is not None:
            x = x + m * moe_ff(rms_norm(x, tensors[p + "norm2"].to(F64), eps), _sub(tensors, p + "mlp."), L["mlp"])
        if side:
            x = token_side(x, tokens, tensors["side.embed"].to(F64), _sub(tensors, p + "side."), i, int(side["dim"]),
                           m, eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    x = rms_norm(x, tensors["final.norm"].to(F64), eps)
    z = (x @ tensors["head"].to(F64).T) * float(config["logit_scale"])
    cap = config.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


def random_weights(config: Dict, seed: int = 0, rel_rows: int = 8) -> Dict[str, torch.Tensor]:
    """Random tensors under the checkpoint's names (float32); ``rel_rows``: rows of every distance table."""
    g = torch.Generator().manual_seed(seed)
    W, V = int(config["width"]), int(config["vocab"])
    side = config.get("token_side")
    n_layers = len(config["layers"])

    def lin(o, i):
        return torch.randn(o, i, generator=g) / math.sqrt(i)

    def gain(n):
        return 1.0 + 0.2 * torch.randn(n, generator=g)

    T = {"embed": torch.randn(V, W, generator=g), "head": lin(V, W), "final.norm": gain(W)}
    if side:
        T["side.embed"] = torch.randn(V, n_layers * int(side["dim"]), generator=g)
    for i, L in enumerate(config["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        T[p + "norm1"] = gain(W)
        for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
            T[p + "mix." + name] = lin(rows, W)
            if int(m.get("conv", 1)) > 1:
                T[p + "mix." + name + ".conv"] = torch.randn(rows, int(m["conv"]), generator=g) * 0.6
        T[p + "mix.q.norm"], T[p + "mix.k.norm"] = gain(d), gain(d)
        T[p + "mix.rel"] = torch.randn(rel_rows, H, generator=g)
        T[p + "mix.g"], T[p + "mix.o"] = lin(H * dv, W), lin(W, H * dv)
        mlp = L.get("mlp")
        if mlp is not None:
            T[p + "norm2"] = gain(W)
            E, Fe = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            T[p + "mlp.router"], T[p + "mlp.router.b"] = lin(E, W) * 2, torch.randn(E, generator=g)
            for e in range(E):
                T[f"{p}mlp.e{e}.up"], T[f"{p}mlp.e{e}.down"] = lin(Fe, W), lin(W, Fe)
            if mlp.get("shared"):
                Fs = int(mlp["shared"]["ff"])
                T[p + "mlp.shared.up"], T[p + "mlp.shared.down"] = lin(Fs, W), lin(W, Fs)
                T[p + "mlp.shared.sg"] = lin(1, W) * 2
        if side:
            ds = int(side["dim"])
            T[p + "side.gate"], T[p + "side.proj"], T[p + "side.norm"] = lin(ds, W), lin(W, ds), gain(W)
    return T
