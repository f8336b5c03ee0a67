"""Serving throughput of a hybrid (Fomalix) stack next to a Llama stack of equal width, depth and feed-forward size, both
through ``InferenceEngineV2.put`` with random weights, plus device times of the hybrid stack's kernels and of their Llama
counterparts against the memory roofline.  ``bench.py --serve`` prints the result as one JSON object.  With
``--serve-model kekopel`` the pair is a Kekopel stack (latent attention with a sliding window, matrix-memory LSTM,
post-scaled layers, dense and expert feed-forwards) next to the Fomalix stack of equal size, and the kernel table sets
every Kekopel kernel beside the Fomalix kernel that does the like job.  With ``--serve-model ridazen`` the pair is a
Ridazen stack (attention with filtered projections, distance-bucket bias and output gate, squared-ReLU experts with a
shared expert, per-layer token input) next to a Fomalix stack of attention layers only at equal size.  With
``--serve-model pifazen`` the pair is a Pifazen stack (latent attention with output gates and scaled rotation, a delta rule
with a decay per key channel, three-power dense feed-forward, clamped experts chosen among groups with identity experts)
next to the Kekopel stack of equal size whose window holds every key.

Timing: CUDA events on the launching stream, >= 3 warm-up forwards, a buffer larger than L2 is rewritten between timed
forwards.  Prefill: one request of ``prefill`` tokens in one forward.  Decode: ``batch`` requests with ``context`` tokens
each advance one token per forward.
"""
from __future__ import annotations

import json
import math
import os
from typing import Callable, Dict, List

import torch

from .config_v2 import RaggedInferenceEngineConfig
from .engine_factory import build_engine_from_model, build_engine_from_state_dict
from .ragged.ragged_manager import DSStateManagerConfig

SIZES = {
    "w1024": dict(width=1024, layers=6, heads=8, kv_heads=2, head=128, ff=4096, ssd_heads=16, ssd_vdim=128, state=128),
    "w2048": dict(width=2048, layers=6, heads=16, kv_heads=4, head=128, ff=8192, ssd_heads=32, ssd_vdim=128, state=128),
    "w4096": dict(width=4096, layers=3, heads=32, kv_heads=8, head=128, ff=14336, ssd_heads=64, ssd_vdim=128, state=128),
}
VOCAB = 32000
CHUNK = 4096          # the prompt and the decode context fall into one chunk: attention work equals full causal


def hybrid_config(z: Dict, kinds=("delta", "mamba2", "attention")) -> Dict:
    mixers = {
        "delta": {"conv": 4, "dim": z["head"], "heads": z["heads"], "kv_heads": z["heads"], "vdim": z["head"]},
        "mamba2": {"conv": 4, "groups": 1, "heads": z["ssd_heads"], "norm_groups": 1, "state": z["state"],
                   "vdim": z["ssd_vdim"]},
        "attention": {"dim": z["head"], "heads": z["heads"], "kv_heads": z["kv_heads"], "mask": {"size": CHUNK},
                      "scale": z["head"] ** -0.5, "vdim": z["head"]},
    }
    layers = [{"type": kinds[i % len(kinds)], "mixer": mixers[kinds[i % len(kinds)]],
               "mlp": {"ff": z["ff"], "kind": "dense"}} for i in range(z["layers"])]
    return {"architecture": "Fomalix", "embedding": {"scale": 1.0}, "layers": layers, "norm": {"eps": 1e-5},
            "vocab": VOCAB, "width": z["width"]}


def hybrid_weights(cfg: Dict, device) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(0)
    W = cfg["width"]

    def mat(o, i):
        return (torch.randn(o, i, generator=g, device=device) / math.sqrt(i)).to(torch.bfloat16)

    def vec(n, lo=0.5, hi=1.5, dt=torch.bfloat16):
        return (torch.rand(n, generator=g, device=device) * (hi - lo) + lo).to(dt)

    out = {"embed": mat(cfg["vocab"], W), "head": mat(cfg["vocab"], W), "final.norm": vec(W)}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            out[p + n] = vec(W)
        ff = L["mlp"]["ff"]
        out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = mat(ff, W), mat(ff, W), mat(W, ff)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, o in (("q", H * d), ("k", G * d), ("v", G * dv)):
                out[p + "mix." + n], out[p + "mix." + n + ".b"] = mat(o, W), vec(o, -0.1, 0.1)
            out[p + "mix.sink"], out[p + "mix.o"] = vec(H, -1, 1), mat(W, H * dv)
        elif L["type"] == "delta":
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, o in (("q", G * d), ("k", G * d), ("v", H * dv)):
                out[p + "mix." + n], out[p + "mix." + n + ".conv"] = mat(o, W), vec(o * taps, -0.5, 0.5).view(o, taps)
            out[p + "mix.b"], out[p + "mix.a"] = mat(H, W), mat(H, W)
            out[p + "mix.A_log"], out[p + "mix.dt_bias"] = vec(H, -2, 0.5), vec(H, -1, 1)
            out[p + "mix.norm"], out[p + "mix.g"], out[p + "mix.o"] = vec(dv), mat(H * dv, W), mat(W, H * dv)
        else:
            H, dv, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = H * dv, H * dv + 2 * G * N
            out[p + "mix.in"] = mat(2 * inner + 2 * G * N + H, W)
            out[p + "mix.conv"], out[p + "mix.conv.b"] = vec(ch * taps, -0.5, 0.5).view(ch, taps), vec(ch, -0.1, 0.1)
            out[p + "mix.dt_bias"], out[p + "mix.A_log"], out[p + "mix.D"] = vec(H, -1, 1), vec(H, -2, 0.5), vec(H)
            out[p + "mix.norm"], out[p + "mix.o"] = vec(inner), mat(W, inner)
    return out


def _engine_config(max_tokens: int, max_seqs: int, pages: int) -> RaggedInferenceEngineConfig:
    sm = DSStateManagerConfig(max_tracked_sequences=max_seqs, max_ragged_sequence_count=max_seqs,
                              max_ragged_batch_size=max(max_tokens, max_seqs), max_context=8192, num_kv_blocks=pages)
    return RaggedInferenceEngineConfig(state_manager=sm, kv_block_size=64)


def build_hybrid(z: Dict, max_tokens: int, max_seqs: int, pages: int):
    cfg = hybrid_config(z)
    return build_engine_from_state_dict(cfg, hybrid_weights(cfg, "cuda"), _engine_config(max_tokens, max_seqs, pages),
                                        dtype=torch.bfloat16)


def build_llama(z: Dict, max_tokens: int, max_seqs: int, pages: int):
    from ...models.llama import LlamaForCausalLM, llama_config
    cfg = llama_config("llama-tiny", hidden_size=z["width"], num_hidden_layers=z["layers"],
                       num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"], intermediate_size=z["ff"],
                       vocab_size=VOCAB, activation_checkpointing=False)
    torch.manual_seed(0)
    lm = LlamaForCausalLM(cfg, device="cuda", dtype=torch.bfloat16).eval()
    return build_engine_from_model(lm, _engine_config(max_tokens, max_seqs, pages))


class _Timer:
    def __init__(self):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")        # > 126 MB of L2

    def __call__(self, fn: Callable[[], None], steps: int, warmup: int) -> float:
        """Median device milliseconds of ``fn``."""
        for _ in range(warmup):
            fn()
        times = []
        for _ in range(steps):
            self.flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        return sorted(times)[len(times) // 2]


def engine_throughput(build, z: Dict, prefill: int, batch: int, context: int, steps: int, warmup: int, timer) -> Dict:
    pages = (prefill + 63) // 64 + batch * ((context + steps + warmup + 8 + 63) // 64) + 8
    eng = build(z, max(prefill, batch, 2048), batch + 1, pages)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, VOCAB, (prefill,), generator=g, dtype=torch.int32)
    uid = [1000]

    def one_prefill():
        uid[0] += 1
        eng.put([uid[0]], [prompt], do_checks=False)
        eng.flush(uid[0])
    ms_p = timer(one_prefill, steps, warmup)
    uids = list(range(batch))
    for lo in range(0, context, 2048):                       # build the contexts, 2048 tokens of one request at a time
        n = min(2048, context - lo)
        for u in uids:
            eng.put([u], [torch.randint(0, VOCAB, (n,), generator=g, dtype=torch.int32)], do_checks=False)
    toks = [torch.randint(0, VOCAB, (1,), generator=g, dtype=torch.int32) for _ in uids]
    ms_d = timer(lambda: eng.put(uids, toks, do_checks=False), steps, warmup)
    del eng
    torch.cuda.empty_cache()
    return {"prefill_tokens": prefill, "prefill_ms": round(ms_p, 3), "prefill_tok_s": round(prefill / ms_p * 1e3),
            "decode_batch": batch, "decode_context": context, "decode_ms": round(ms_d, 3),
            "decode_tok_s": round(batch / ms_d * 1e3)}


def kernel_table(z: Dict, prefill: int, batch: int, context: int, timer, hbm_gbs: float,
                 peak_tflops: Dict[str, float]) -> List[Dict]:
    """Device time, algorithmic bytes and fraction of the copy bandwidth for the hybrid stack's kernels and the Llama
    kernels that do the like job, at prefill (one request) and decode (``batch`` requests) shapes."""
    from ...ops import functional as F
    from .kernels import mixer_ops as M
    from .kernels import ragged_ops as R
    from .ragged.ragged_wrapper import RaggedBatchWrapper
    dev, bf = "cuda", torch.bfloat16
    W, H, G, d = z["width"], z["heads"], z["kv_heads"], z["head"]
    Hs, dvs, N = z["ssd_heads"], z["ssd_vdim"], z["state"]
    rows: List[Dict] = []

    def add(name, phase, fn, nbytes, flops=0.0, pipe=None):
        """``pipe``: the arithmetic unit the kernel's products run on ("fp32": FMA lanes, "bf16": tensor cores); the
        roofline time is the larger of bytes / copy bandwidth and FLOPs / that unit's peak."""
        ms = timer(fn, 5, 3)
        ideal_ms = nbytes / hbm_gbs / 1e6
        if pipe is not None:
            ideal_ms = max(ideal_ms, flops / peak_tflops[pipe] / 1e9)
        rows.append({"kernel": name, "phase": phase, "ms": round(ms, 4), "GB_s": round(nbytes / ms / 1e6, 1),
                     "of_measured_hbm": round(nbytes / ms / 1e6 / hbm_gbs, 3), "GFLOP_s": round(flops / ms / 1e6, 1),
                     "pipe": pipe or "memory", "of_roofline": round(ideal_ms / ms, 3)})

    for phase, T, n_seq, seen in (("prefill", prefill, 1, 0), ("decode", batch, batch, context)):
        per = T // n_seq
        tot = seen + per
        n_pages_seq = (tot + 63) // 64
        t2s = torch.arange(n_seq, device=dev, dtype=torch.int32).repeat_interleave(per)
        pos = (torch.arange(per, device=dev, dtype=torch.int32) + seen).repeat(n_seq)
        tables = torch.arange(n_seq * n_pages_seq, device=dev, dtype=torch.int32).view(n_seq, n_pages_seq)
        info = torch.tensor([[i * per, per, seen, i] for i in range(n_seq)], dtype=torch.int32, device=dev)
        resid = torch.randn(T, W, device=dev)
        y = torch.randn(T, W, device=dev).to(bf)
        w = torch.ones(W, device=dev, dtype=bf)
        add("resid_norm_step (post-norm + add + pre-norm)", phase,
            lambda: M.resid_norm_step(resid, y, w, None, w, 1e-5, bf), T * W * (4 + 4 + 2 + 2))
        add("llama rms_norm with residual add", phase, lambda: F.rms_norm(y, w, 1e-5, y), T * W * 2 * 4)
        # attention: append + attend
        qkv = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
        bias = torch.zeros((H + 2 * G) * d, device=dev, dtype=bf)
        kc = torch.randn(n_seq * n_pages_seq, 64, G, d, device=dev).to(bf)
        vc = torch.randn(n_seq * n_pages_seq, 64, G, d, device=dev).to(bf)
        sink = torch.zeros(H, device=dev)
        add("qk_norm_append", phase,
            lambda: M.qk_norm_append(qkv, bias, kc, vc, t2s, pos, tables, H, G, d, d, 1e-5, True),
            T * ((H + 2 * G) * d * 2 + H * d * 4 + 2 * G * d * 2))
        q32 = torch.randn(T, H, d, device=dev)
        lo = (seen + per - 1) // CHUNK * CHUNK
        keys_per_q = (min(per, CHUNK) + 1) / 2 if phase == "prefill" else (tot - lo)
        kv_bytes = n_seq * (tot if phase == "prefill" else tot - lo) * 2 * G * d * 2
        fl = 4.0 * T * H * d * keys_per_q
        cache = torch.randn(n_seq * n_pages_seq, 64, 2, G, d, device=dev).to(bf)
        add("llama kv_rotary_blocked", phase,
            lambda: R.kv_rotary_blocked(qkv, cache, t2s, pos, tables, H, G, d, d, 10000.0),
            T * ((H + 2 * G) * d * 2 * 2 + 2 * G * d * 2))
        wrap = RaggedBatchWrapper(max(T, 64), n_seq, n_pages_seq, device=dev)

        class _Seq:
            def __init__(self, i):
                self.seen_tokens, self._b = seen, tables[i].cpu()

            def kv_blocks(self):
                return self._b
        for i in range(n_seq):
            wrap.insert_sequence(_Seq(i), torch.zeros(per, dtype=torch.int32), do_checks=False)
        wrap.finalize()
        atoms, n_long = wrap.atoms(), wrap.atoms_longer_than(M.SHORT_ATOM)
        add(f"sink_attention (chunk {CHUNK}, fp32 weights)", phase,
            lambda: M.sink_attention(q32, kc, vc, sink, t2s, pos, tables, d ** -0.5, CHUNK, bf, atoms, n_long),
            kv_bytes + T * H * d * 6, fl, "fp32")
        qv = qkv.view(T, H + 2 * G, d)[:, :H]
        full_keys = (per + 1) / 2 if phase == "prefill" else tot
        add("llama ragged_attention (full causal)", phase, lambda: R.ragged_attention(qv, cache, wrap),
            n_seq * tot * 2 * G * d * 2 + T * H * d * 4, 4.0 * T * H * d * full_keys, "bf16")
        # recurrences
        for name, Hh, Gg, n, dv, delta in (("delta", H, H, d, d, True), ("ssd", Hs, 1, N, dvs, False)):
            C = (2 * Gg * n + Hh * dv)
            x = torch.randn(T, C, device=dev).to(bf)
            cw = torch.randn(C, 4, device=dev).to(bf)
            cst = torch.zeros(n_seq, 3, C, device=dev, dtype=bf)
            add(f"conv_silu + state update ({name} channels)", phase,
                lambda: (M.conv_silu(x, cw, None, cst, info, t2s), M.conv_state_update(x, cst, info)),
                T * C * (2 + 4) + n_seq * 3 * C * 4)
            xc = torch.randn(T, C, device=dev)
            xc[:, : 2 * Gg * n] /= math.sqrt(n)
            decay, beta = torch.rand(T, Hh, device=dev) * 0.1 + 0.9, torch.rand(T, Hh, device=dev)
            S = torch.zeros(n_seq, Hh, dv, n, device=dev)
            state_bytes = n_seq * Hh * dv * n * 4 * (2 if seen else 1)
            add(f"linear_recurrence ({name})", phase,
                lambda: M.linear_recurrence(xc[:, : Gg * n], xc[:, Gg * n: 2 * Gg * n], xc[:, 2 * Gg * n:], decay, beta,
                                            None, S, info, Hh, Gg, n, dv, delta),
                state_bytes + T * (C * 4 + Hh * dv * 4), (6.0 if delta else 4.0) * T * Hh * dv * n, "fp32")
            o = torch.randn(T, Hh * dv, device=dev)
            gate = torch.randn(T, Hh * dv, device=dev).to(bf)
            nw = torch.ones(dv if delta else Hh * dv, device=dev, dtype=bf)
            add(f"group_norm_gate ({name})", phase,
                lambda: M.group_norm_gate(o, gate, nw, dv if delta else Hh * dv, 1e-5, not delta, bf),
                T * Hh * dv * (4 + 2 + 2))
    return rows


# ------------------------------------------------------------------------------------------------ Kekopel beside Fomalix
WINDOW = 1024         # sliding window of the latent attention layers
LATENT = dict(q_rank=512, kv_rank=192, rot=64)      # the cached row is kv_rank + rot = 256 channels


def kekopel_config(z: Dict) -> Dict:
    kinds = ["latent_attention", "mlstm", "latent_attention"]
    mixers = {
        "latent_attention": {"dim": z["head"], "heads": z["heads"], "kv_rank": LATENT["kv_rank"],
                             "mask": {"size": WINDOW}, "q_rank": LATENT["q_rank"],
                             "rot": {"base": 10000.0, "dims": LATENT["rot"]}, "rot_dim": LATENT["rot"],
                             "scale": (z["head"] + LATENT["rot"]) ** -0.5, "vdim": z["head"]},
        "mlstm": {"dim": z["head"], "gate_cap": 15.0, "heads": z["heads"], "vdim": z["head"]},
    }
    mlps = [{"ff": z["ff"], "kind": "dense"},
            {"expert": {"ff": z["ff"] // 4}, "kind": "moe", "router": {"experts": 8, "top": 2}}]
    layers = [{"type": kinds[i % 3], "mixer": mixers[kinds[i % 3]], "mlp": mlps[i % 2]} for i in range(z["layers"])]
    return {"architecture": "Kekopel", "canon": {"taps": 4}, "layers": layers, "norm": {"eps": 1e-5}, "vocab": VOCAB,
            "width": z["width"]}


def kekopel_weights(cfg: Dict, device) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(0)
    W = cfg["width"]
    bf = torch.bfloat16

    def mat(o, i):
        return (torch.randn(o, i, generator=g, device=device) / math.sqrt(i)).to(bf)

    def vec(n, lo=0.5, hi=1.5):
        return (torch.rand(n, generator=g, device=device) * (hi - lo) + lo).to(bf)

    out = {"embed": mat(cfg["vocab"], W), "head": mat(cfg["vocab"], W), "final.norm": vec(1).reshape(())}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        for n in ("1", "2"):
            out[p + "norm" + n], out[p + "ls" + n] = vec(1).reshape(()), vec(W, 0.2, 0.8)
            out[p + "canon" + n] = vec(W * 4, -0.3, 0.3).view(W, 4)
        out[p + "dwa"] = torch.cat([vec(i + 1, -0.1, 0.1), vec(1, 0.8, 1.0)])
        if L["type"] == "latent_attention":
            H, d, rot, dv, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out[p + "mix.dq"], out[p + "mix.dq.norm"], out[p + "mix.uq"] = mat(qr, W), vec(qr), mat(H * (d + rot), qr)
            out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = mat(r + rot, W), vec(r)
            out[p + "mix.uk"], out[p + "mix.uv"] = mat(H * d, r), mat(H * dv, r)
            out[p + "mix.sink"], out[p + "mix.o"] = vec(H, -1, 1), mat(W, H * dv)
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            for n, o in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv), ("i", H), ("f", H)):
                out[p + "mix." + n] = mat(o, W)
            out[p + "mix.i.b"], out[p + "mix.f.b"] = vec(H, -3, -1), vec(H, 2, 4)
            out[p + "mix.norm"], out[p + "mix.o"] = vec(H * dv), mat(W, H * dv)
        mlp = L["mlp"]
        if mlp["kind"] == "dense":
            out[p + "mlp.up"], out[p + "mlp.up.b"] = mat(mlp["ff"], W), vec(mlp["ff"], -0.1, 0.1)
            out[p + "mlp.down"], out[p + "mlp.down.b"] = mat(W, mlp["ff"]), vec(W, -0.1, 0.1)
        else:
            F_ = mlp["expert"]["ff"]
            out[p + "mlp.router"] = mat(mlp["router"]["experts"], W)
            for e in range(mlp["router"]["experts"]):
                out[p + f"mlp.e{e}.gate"], out[p + f"mlp.e{e}.up"] = mat(F_, W), mat(F_, W)
                out[p + f"mlp.e{e}.down"] = mat(W, F_)
    return out


def build_kekopel(z: Dict, max_tokens: int, max_seqs: int, pages: int):
    cfg = kekopel_config(z)
    return build_engine_from_state_dict(cfg, kekopel_weights(cfg, "cuda"), _engine_config(max_tokens, max_seqs, pages),
                                        dtype=torch.bfloat16)


def kekopel_kernel_table(z: Dict, prefill: int, batch: int, context: int, timer, hbm_gbs: float,
                         peak_tflops: Dict[str, float]) -> List[Dict]:
    """Every Kekopel kernel beside the Fomalix kernel that does the like job (``like``), at prefill (one request) and
    decode (``batch`` requests) shapes: device time, algorithmic bytes and FLOPs, fraction of the roofline (the larger
    of bytes / copy bandwidth and FLOPs / the peak of the unit the products run on)."""
    from ...moe import fused_ep
    from ...ops import functional as F
    from ...ops import moe_ops
    from .kernels import mixer_ops as M
    from .ragged.ragged_wrapper import RaggedBatchWrapper
    dev, bf = "cuda", torch.bfloat16
    W, H, G, d, ff = z["width"], z["heads"], z["kv_heads"], z["head"], z["ff"]
    r, rot, qr = LATENT["kv_rank"], LATENT["rot"], LATENT["q_rank"]
    rows: List[Dict] = []

    def add(name, like, phase, fn, nbytes, flops=0.0, pipe=None):
        ms = timer(fn, 5, 3)
        ideal_ms = nbytes / hbm_gbs / 1e6
        if pipe is not None:
            ideal_ms = max(ideal_ms, flops / peak_tflops[pipe] / 1e9)
        rows.append({"kernel": name, "like": like, "phase": phase, "ms": round(ms, 4),
                     "GB_s": round(nbytes / ms / 1e6, 1), "GFLOP_s": round(flops / ms / 1e6, 1), "pipe": pipe or "memory",
                     "of_roofline": round(ideal_ms / ms, 3)})

    for phase, T, n_seq, seen in (("prefill", prefill, 1, 0), ("decode", batch, batch, context)):
        per = T // n_seq
        tot = seen + per
        n_pages_seq = (tot + 63) // 64
        t2s = torch.arange(n_seq, device=dev, dtype=torch.int32).repeat_interleave(per)
        pos = (torch.arange(per, device=dev, dtype=torch.int32) + seen).repeat(n_seq)
        tables = torch.arange(n_seq * n_pages_seq, device=dev, dtype=torch.int32).view(n_seq, n_pages_seq)
        info = torch.tensor([[i * per, per, seen, i] for i in range(n_seq)], dtype=torch.int32, device=dev)
        x32 = torch.randn(T, W, device=dev)
        y = torch.randn(T, W, device=dev).to(bf)
        wv = torch.ones(W, device=dev, dtype=bf)
        # stream: filter in front of a sublayer, post-norm (+ mixture of 4 streams) behind it
        cw = torch.randn(W, 4, device=dev).to(bf)
        cst = torch.zeros(n_seq, 3, W, device=dev)
        add("conv_residual + state update", None, phase,
            lambda: (M.conv_residual(x32, cw, cst, info, t2s, bf), M.conv_state_update(x32, cst, info)),
            T * W * (4 + 2) + n_seq * 3 * W * 4 * 2)
        xb = x32.to(bf)
        cstb = torch.zeros(n_seq, 3, W, device=dev, dtype=bf)
        add("conv_silu + state update", "conv_residual + state update", phase,
            lambda: (M.conv_silu(xb, cw, None, cstb, info, t2s), M.conv_state_update(xb, cstb, info)),
            T * W * (2 + 4) + n_seq * 3 * W * 2 * 2)
        gain, ls = torch.ones(1, device=dev), torch.ones(W, device=dev)
        stack = torch.randn(5, T, W, device=dev)
        mixw, mixed = torch.ones(5, device=dev), torch.empty(T, W, device=dev)
        add("post_norm_mix (no mixture)", None, phase,
            lambda: M.post_norm_mix(x32, y, gain, ls, stack[4], 1e-5), T * W * (4 + 2 + 4))
        add("post_norm_mix (mixture of 5 streams)", None, phase,
            lambda: M.post_norm_mix(x32, y, gain, ls, stack[4], 1e-5, stack, 4, mixw, mixed), T * W * (4 + 2 + 4 + 4 * 4 + 4))
        add("resid_norm_step", "post_norm_mix (no mixture)", phase,
            lambda: M.resid_norm_step(x32, y, wv, None, wv, 1e-5, bf), T * W * (4 + 4 + 2 + 2))
        # latent attention: prepare + attend
        proj = torch.randn(T, qr + r + rot, device=dev).to(bf)
        qn = torch.ones(qr, device=dev, dtype=bf)
        add("rms_norm_slice (query latent)", None, phase, lambda: M.rms_norm_slice(proj[:, :qr], qn, 1e-5), T * qr * 4)
        q = torch.randn(T, H * (d + rot), device=dev).to(bf)
        q_abs = torch.randn(H, T, r, device=dev).to(bf).transpose(0, 1)
        kn = torch.ones(r, device=dev, dtype=bf)
        inv = torch.pow(torch.tensor(10000.0), -torch.arange(0, rot, 2, dtype=torch.float32) / rot).to(dev)
        cache = torch.randn(n_seq * n_pages_seq, 64, 1, r + rot, device=dev).to(bf)
        add("latent_qk_prepare", None, phase,
            lambda: M.latent_qk_prepare(q, q_abs, proj[:, qr:], kn, inv, cache, t2s, pos, tables, H, d, rot, 1e-5),
            T * ((r + rot) * 4 + H * (r + rot) * (2 + 4)))
        qkv = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
        bias = torch.zeros((H + 2 * G) * d, device=dev, dtype=bf)
        kc = torch.randn(n_seq * n_pages_seq, 64, G, d, device=dev).to(bf)
        vc = torch.randn(n_seq * n_pages_seq, 64, G, d, device=dev).to(bf)
        add("qk_norm_append", "latent_qk_prepare", phase,
            lambda: M.qk_norm_append(qkv, bias, kc, vc, t2s, pos, tables, H, G, d, d, 1e-5, True),
            T * ((H + 2 * G) * d * 2 + H * d * 4 + 2 * G * d * 2))
        wrap = RaggedBatchWrapper(max(T, 64), n_seq, n_pages_seq, device=dev)

        class _Seq:
            def __init__(self, i):
                self.seen_tokens, self._b = seen, tables[i].cpu()

            def kv_blocks(self):
                return self._b
        for i in range(n_seq):
            wrap.insert_sequence(_Seq(i), torch.zeros(per, dtype=torch.int32), do_checks=False)
        wrap.finalize()
        atoms, n_long = wrap.atoms(), wrap.atoms_longer_than(M.SHORT_ATOM)
        sink = torch.zeros(H, device=dev)
        ql = torch.randn(T, H, r + rot, device=dev)
        if phase == "prefill":
            keys_per_q = sum(min(p + 1, WINDOW) for p in range(per)) / per
            keys_read = n_seq * tot
        else:
            keys_per_q = min(tot, WINDOW)
            keys_read = n_seq * min(tot, WINDOW)
        add(f"sink_attention, latent rows (window {WINDOW})", None, phase,
            lambda: M.sink_attention(ql, cache, None, sink, t2s, pos, tables, 0.06, 0, bf, atoms, n_long, window=WINDOW,
                                     value_cols=r),
            keys_read * (r + rot) * 2 + T * H * ((r + rot) * 4 + r * 2), 2.0 * T * H * (2 * r + rot) * keys_per_q, "fp32")
        q32 = torch.randn(T, H, d, device=dev)
        add(f"sink_attention, per-head keys (chunk {WINDOW})", f"sink_attention, latent rows (window {WINDOW})", phase,
            lambda: M.sink_attention(q32, kc, vc, sink, t2s, pos, tables, d ** -0.5, WINDOW, bf, atoms, n_long),
            n_seq * (tot if phase == "prefill" else (tot - (tot - 1) // WINDOW * WINDOW)) * 2 * G * d * 2 + T * H * d * 6,
            4.0 * T * H * d * ((min(per, WINDOW) + 1) / 2 if phase == "prefill" else (tot - (tot - 1) // WINDOW * WINDOW)),
            "fp32")
        # matrix-memory LSTM beside the state-space recurrence of the same head count and sizes
        Pw = 2 * H * d + 2 * H * d + 2 * H
        pm = torch.randn(T, (Pw + 7) // 8 * 8, device=dev).to(bf)
        bi, bfg = torch.zeros(H, device=dev), torch.ones(H, device=dev)
        mst = torch.zeros(n_seq, H, device=dev)
        i0 = 4 * H * d
        add("mlstm_gate_scan", None, phase,
            lambda: M.mlstm_gate_scan(pm[:, i0: i0 + H], pm[:, i0 + H: i0 + 2 * H], bi, bfg, 15.0, mst, info),
            T * H * (2 * 2 + 3 * 4))
        A_log, dtb = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
        add("recurrence_gates", "mlstm_gate_scan", phase,
            lambda: M.recurrence_gates(pm[:, i0: i0 + H], pm[:, i0 + H: i0 + 2 * H], A_log, dtb, "delta"),
            T * H * (2 * 2 + 2 * 4))
        add("mlstm_prepare", None, phase, lambda: M.mlstm_prepare(pm, H, d, d, d ** -0.5),
            T * (3 * H * d * 2 + (3 * H * d + H) * 4))
        xm = M.mlstm_prepare(pm, H, d, d, d ** -0.5)
        xm[:, : 2 * H * d] /= math.sqrt(d)
        decay, beta = torch.rand(T, H, device=dev) * 0.1 + 0.9, torch.rand(T, H, device=dev)
        S1 = torch.zeros(n_seq, H, d + 1, d, device=dev)
        sb = (2 if seen else 1) * 4
        add("linear_recurrence (mlstm, values + normaliser)", None, phase,
            lambda: M.linear_recurrence(xm[:, H * d: 2 * H * d], xm[:, : H * d], xm[:, 2 * H * d:], decay, beta, None, S1,
                                        info, H, H, d, d + 1, False),
            n_seq * H * (d + 1) * d * sb + T * ((3 * H * d + H) * 4 + H * (d + 1) * 4), 4.0 * T * H * (d + 1) * d, "fp32")
        xs = torch.randn(T, 3 * H * d, device=dev)
        xs[:, : 2 * H * d] /= math.sqrt(d)
        S0 = torch.zeros(n_seq, H, d, d, device=dev)
        add("linear_recurrence (same sizes, no normaliser)", "linear_recurrence (mlstm, values + normaliser)", phase,
            lambda: M.linear_recurrence(xs[:, H * d: 2 * H * d], xs[:, : H * d], xs[:, 2 * H * d:], decay, beta, None, S0,
                                        info, H, H, d, d, False),
            n_seq * H * d * d * sb + T * (3 * H * d * 4 + H * d * 4), 4.0 * T * H * d * d, "fp32")
        o1 = torch.randn(T, H * (d + 1), device=dev)
        mt = torch.zeros(T, H, device=dev)
        gate = torch.randn(T, H * d, device=dev).to(bf)
        nw = torch.ones(H * d, device=dev, dtype=bf)
        add("mlstm_output", None, phase, lambda: M.mlstm_output(o1, mt, gate, nw, H, d, 1e-5, bf),
            T * H * ((d + 1) * 4 + d * (2 + 2)))
        o0 = torch.randn(T, H * d, device=dev)
        add("group_norm_gate", "mlstm_output", phase, lambda: M.group_norm_gate(o0, gate, nw[:d], d, 1e-5, False, bf),
            T * H * d * (4 + 2 + 2))
        # feed-forwards
        hu = torch.randn(T, ff, device=dev).to(bf)
        bu = torch.zeros(ff, device=dev, dtype=bf)
        add("bias_act_rows (squared relu)", None, phase, lambda: M.bias_act_rows(hu, bu, "relu_sq"), T * ff * 4)
        hg = torch.randn(T, 2 * ff, device=dev).to(bf)
        add("gated_act", "bias_act_rows (squared relu)", phase, lambda: F.gated_act(hg, "gelu"), T * ff * 6)
        E, K, Fe = 8, 2, ff // 4
        logits = torch.randn(T, E, device=dev)
        xe = torch.randn(T, W, device=dev).to(bf)
        w1 = (torch.randn(E, 2 * Fe, W, device=dev) / math.sqrt(W)).to(bf)
        w2 = (torch.randn(E, W, Fe, device=dev) / math.sqrt(Fe)).to(bf)
        moe_bytes = E * 3 * Fe * W * 2 + T * W * 2 * (1 + 2 * K + 1) + T * K * 3 * Fe * 2
        moe_flops = 2.0 * T * K * 3 * Fe * W

        def experts(score_function, weight_input):
            s, a, o, c = moe_ops.top_k_gating(logits, K, renormalize=False, score_function=score_function)
            return fused_ep.grouped_experts_inference(xe, s, a, o, c, w1, w2, F.swiglu, K, weight_input=weight_input)
        add("experts: sigmoid gating, weighted rows in, grouped GEMMs, plain sum", None, phase,
            lambda: experts("sigmoid", True), moe_bytes, moe_flops, "bf16")
        add("experts: softmax gating, rows in, grouped GEMMs, weighted sum", "experts: sigmoid gating, weighted rows in, "
            "grouped GEMMs, plain sum", phase, lambda: experts("softmax", False), moe_bytes, moe_flops, "bf16")
    by_name = {(r_["kernel"], r_["phase"]): r_ for r_ in rows}
    for r_ in rows:                      # distance from the roofline relative to the like kernel's
        if r_["like"]:
            mine = by_name[(r_["like"], r_["phase"])]
            mine["like_of_roofline"] = r_["of_roofline"]
            mine["like_kernel"] = r_["kernel"]
    return rows


# ------------------------------------------------------------------------------------------------ Ridazen beside Fomalix
RIDAZEN = dict(taps=4, rows=32, far=1024, every=64, coef=0.1, experts=8, top=2, side=64)


def ridazen_config(z: Dict) -> Dict:
    mixer = {"bias_max": RIDAZEN["far"], "conv": RIDAZEN["taps"], "dim": z["head"], "heads": z["heads"],
             "kv_heads": z["kv_heads"], "q_temp": {"coef": RIDAZEN["coef"], "every": RIDAZEN["every"]},
             "scale": z["head"] ** -0.5, "vdim": z["head"]}
    mlp = {"expert": {"ff": z["ff"] // 4}, "kind": "moe", "router": {"experts": RIDAZEN["experts"], "top": RIDAZEN["top"]},
           "shared": {"ff": z["ff"] // 4}}
    return {"architecture": "Ridazen", "layers": [{"type": "attention", "mixer": mixer, "mlp": mlp}] * z["layers"],
            "logit_scale": 0.5, "logit_softcap": 30.0, "loop": None, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "token_side": {"dim": RIDAZEN["side"]}, "vocab": VOCAB, "width": z["width"]}


def ridazen_weights(cfg: Dict, device) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(0)
    W, bf = cfg["width"], torch.bfloat16

    def mat(o, i):
        return (torch.randn(o, i, generator=g, device=device) / math.sqrt(i)).to(bf)

    def vec(n, lo=0.5, hi=1.5):
        return (torch.rand(n, generator=g, device=device) * (hi - lo) + lo).to(bf)

    ds = cfg["token_side"]["dim"]
    out = {"embed": mat(cfg["vocab"], W), "head": mat(cfg["vocab"], W), "final.norm": vec(W),
           "side.embed": mat(cfg["vocab"], len(cfg["layers"]) * ds)}
    for i, L in enumerate(cfg["layers"]):
        m, mlp, p = L["mixer"], L["mlp"], f"l{i}."
        H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        out[p + "norm1"], out[p + "norm2"] = vec(W), vec(W)
        for n, o in (("q", H * d), ("k", G * d), ("v", G * dv)):
            out[p + "mix." + n], out[p + "mix." + n + ".conv"] = mat(o, W), vec(o * taps, -0.5, 0.5).view(o, taps)
        out[p + "mix.q.norm"], out[p + "mix.k.norm"] = vec(d), vec(d)
        out[p + "mix.rel"] = vec(RIDAZEN["rows"] * H, -1, 1).view(RIDAZEN["rows"], H)
        out[p + "mix.g"], out[p + "mix.o"] = mat(H * dv, W), mat(W, H * dv)
        Fe, Fs, E = mlp["expert"]["ff"], mlp["shared"]["ff"], mlp["router"]["experts"]
        out[p + "mlp.router"], out[p + "mlp.router.b"] = mat(E, W), vec(E, -0.5, 0.5)
        for e in range(E):
            out[p + f"mlp.e{e}.up"], out[p + f"mlp.e{e}.down"] = mat(Fe, W), mat(W, Fe)
        out[p + "mlp.shared.up"], out[p + "mlp.shared.down"] = mat(Fs, W), mat(W, Fs)
        out[p + "mlp.shared.sg"] = mat(1, W)
        out[p + "side.gate"], out[p + "side.proj"], out[p + "side.norm"] = mat(ds, W), mat(W, ds), vec(W)
    return out


def build_ridazen(z: Dict, max_tokens: int, max_seqs: int, pages: int):
    cfg = ridazen_config(z)
    return build_engine_from_state_dict(cfg, ridazen_weights(cfg, "cuda"), _engine_config(max_tokens, max_seqs, pages),
                                        dtype=torch.bfloat16)


def build_attention_stack(z: Dict, max_tokens: int, max_seqs: int, pages: int):
    """The Fomalix stack with attention layers only (per-head keys, sink, dense gated feed-forward)."""
    cfg = hybrid_config(z, kinds=("attention",))
    return build_engine_from_state_dict(cfg, hybrid_weights(cfg, "cuda"), _engine_config(max_tokens, max_seqs, pages),
                                        dtype=torch.bfloat16)


def ridazen_kernel_table(z: Dict, prefill: int, batch: int, context: int, timer, hbm_gbs: float,
                         peak_tflops: Dict[str, float]) -> List[Dict]:
    """Every Ridazen kernel beside the kernel of the Fomalix (or Kekopel) stack that does the like job (``like``), at
    prefill (one request) and decode (``batch`` requests) shapes: device time, algorithmic bytes and FLOPs, fraction
    of the roofline (the larger of bytes / copy bandwidth and FLOPs / the peak of the unit the products run on)."""
    from ...moe import fused_ep
    from ...ops import functional as F
    from ...ops import moe_ops
    from .kernels import mixer_ops as M
    from .modules.implementations import DSFilteredBiasAttention
    from .ragged.ragged_wrapper import RaggedBatchWrapper
    dev, bf = "cuda", torch.bfloat16
    W, H, G, d, ff = z["width"], z["heads"], z["kv_heads"], z["head"], z["ff"]
    taps, ds = RIDAZEN["taps"], RIDAZEN["side"]
    rows: List[Dict] = []

    def add(name, like, phase, fn, nbytes, flops=0.0, pipe=None):
        ms = timer(fn, 5, 3)
        ideal_ms = nbytes / hbm_gbs / 1e6
        if pipe is not None:
            ideal_ms = max(ideal_ms, flops / peak_tflops[pipe] / 1e9)
        rows.append({"kernel": name, "like": like, "phase": phase, "ms": round(ms, 4),
                     "GB_s": round(nbytes / ms / 1e6, 1), "GFLOP_s": round(flops / ms / 1e6, 1), "pipe": pipe or "memory",
                     "of_roofline": round(ideal_ms / ms, 3)})

    for phase, T, n_seq, seen in (("prefill", prefill, 1, 0), ("decode", batch, batch, context)):
        per = T // n_seq
        tot = seen + per
        n_pages_seq = (tot + 63) // 64
        t2s = torch.arange(n_seq, device=dev, dtype=torch.int32).repeat_interleave(per)
        pos = (torch.arange(per, device=dev, dtype=torch.int32) + seen).repeat(n_seq)
        tables = torch.arange(n_seq * n_pages_seq, device=dev, dtype=torch.int32).view(n_seq, n_pages_seq)
        info = torch.tensor([[i * per, per, seen, i] for i in range(n_seq)], dtype=torch.int32, device=dev)
        x32 = torch.randn(T, W, device=dev)
        y = torch.randn(T, W, device=dev).to(bf)
        wv = torch.ones(W, device=dev, dtype=bf)
        add("resid_norm_step (scaled add + pre-norm)", None, phase,
            lambda: M.resid_norm_step(x32, y, None, None, wv, 1e-5, bf, 0.5), T * W * (4 + 4 + 2 + 2))
        add("resid_norm_step (scaled add + 16-bit copy)", None, phase,
            lambda: M.resid_norm_step(x32, y, None, None, None, 1e-5, bf, 0.5, copy_out=True), T * W * (4 + 4 + 2 + 2))
        add("resid_norm_step (post-norm + add + pre-norm)", "resid_norm_step (scaled add + pre-norm)", phase,
            lambda: M.resid_norm_step(x32, y, wv, None, wv, 1e-5, bf), T * W * (4 + 4 + 2 + 2))
        # projections -> filter -> norm -> cache
        C = (H + 2 * G) * d
        proj = torch.randn(T, C + H * d, device=dev).to(bf)
        cw = (torch.randn(C, taps, device=dev) * 0.3).to(bf)
        cst = torch.zeros(n_seq, taps - 1, C, device=dev, dtype=bf)
        nq = torch.ones(d, device=dev, dtype=bf)
        kc = torch.randn(n_seq * n_pages_seq, 64, G, d, device=dev).to(bf)
        vc = torch.randn(n_seq * n_pages_seq, 64, G, d, device=dev).to(bf)
        add("qkv_filter_norm_append + state update", None, phase,
            lambda: (M.qkv_filter_norm_append(proj, cw, cst, info, nq, nq, kc, vc, t2s, pos, tables, H, G, d, d, 1e-5,
                                              True, RIDAZEN["coef"], RIDAZEN["every"]),
                     M.conv_state_update(proj[:, :C], cst, info)),
            T * (C * 2 + H * d * 4 + 2 * G * d * 2) + n_seq * (taps - 1) * C * 2 * 2)
        qkv = torch.randn(T, C, device=dev).to(bf)
        bias = torch.zeros(C, device=dev, dtype=bf)
        add("qk_norm_append", "qkv_filter_norm_append + state update", phase,
            lambda: M.qk_norm_append(qkv, bias, kc, vc, t2s, pos, tables, H, G, d, d, 1e-5, True),
            T * (C * 2 + H * d * 4 + 2 * G * d * 2))
        wrap = RaggedBatchWrapper(max(T, 64), n_seq, n_pages_seq, device=dev)

        class _Seq:
            def __init__(self, i):
                self.seen_tokens, self._b = seen, tables[i].cpu()

            def kv_blocks(self):
                return self._b
        for i in range(n_seq):
            wrap.insert_sequence(_Seq(i), torch.zeros(per, dtype=torch.int32), do_checks=False)
        wrap.finalize()
        atoms, n_long = wrap.atoms(), wrap.atoms_longer_than(M.SHORT_ATOM)
        q32 = torch.randn(T, H, d, device=dev)
        table = torch.randn(RIDAZEN["rows"], H, device=dev)
        dist = DSFilteredBiasAttention.expand_distance_bias(table, RIDAZEN["far"])
        gate = proj[:, C:]
        keys_per_q = (per + 1) / 2 if phase == "prefill" else tot
        kv_bytes = n_seq * tot * 2 * G * d * 2
        fl = 4.0 * T * H * d * keys_per_q
        add("sink_attention (causal, distance bias, output gate)", None, phase,
            lambda: M.sink_attention(q32, kc, vc, None, t2s, pos, tables, d ** -0.5, 0, bf, atoms, n_long, dist_bias=dist,
                                     gate=gate), kv_bytes + T * H * d * 8, fl, "fp32")
        sink = torch.zeros(H, device=dev)
        add("sink_attention (causal, sink)", "sink_attention (causal, distance bias, output gate)", phase,
            lambda: M.sink_attention(q32, kc, vc, sink, t2s, pos, tables, d ** -0.5, 0, bf, atoms, n_long),
            kv_bytes + T * H * d * 6, fl, "fp32")
        # per-layer token input and logits
        dsp = (ds + 7) // 8 * 8
        gx = torch.randn(T, dsp, device=dev).to(bf)
        side = torch.randn(VOCAB, 6 * ds, device=dev).to(bf)
        ids = torch.randint(0, VOCAB, (T,), device=dev, dtype=torch.int32)
        add("side_gate", None, phase, lambda: M.side_gate(gx, side, ids, 2 * ds, ds, dsp), T * ds * 6)
        hg = torch.randn(T, 2 * dsp, device=dev).to(bf)
        add("gated_act_rows", "side_gate", phase, lambda: M.gated_act_rows(hg, "gelu"), T * dsp * 6)
        # feed-forward
        E, K, Fe = RIDAZEN["experts"], RIDAZEN["top"], ff // 4
        hu = torch.randn(T, Fe, device=dev).to(bf)
        add("bias_act_rows (squared relu, shared expert)", None, phase, lambda: M.bias_act_rows(hu, None, "relu_sq"),
            T * Fe * 4)
        hgu = torch.randn(T, 2 * Fe, device=dev).to(bf)
        add("gated_act", "bias_act_rows (squared relu, shared expert)", phase, lambda: F.gated_act(hgu, "gelu"), T * Fe * 6)
        acc = torch.randn(T, W, device=dev).to(bf)
        sg = torch.randn(T, E + 1, device=dev)
        add("row_gate_add (shared expert into the experts' sum)", None, phase,
            lambda: M.row_gate_add_(acc, y, sg[:, E]), T * W * 6)
        add("bias_act_rows (same rows)", "row_gate_add (shared expert into the experts' sum)", phase,
            lambda: M.bias_act_rows(acc, wv, "identity"), T * W * 4)
        logits = torch.randn(T, E, device=dev)
        xe = torch.randn(T, W, device=dev).to(bf)
        wr, br = torch.randn(E + 1, W, device=dev) / math.sqrt(W), torch.zeros(E + 1, device=dev)
        add("router_logits (16-bit rows x fp32 weights, experts + shared gate)", None, phase,
            lambda: M.router_logits(xe, wr, br), T * W * 2 + (E + 1) * W * 4 + T * (E + 1) * 4)
        add("32-bit copy of the rows + library product", "router_logits (16-bit rows x fp32 weights, experts + shared gate)",
            phase, lambda: torch.nn.functional.linear(xe.float(), wr, br), T * W * 2 + (E + 1) * W * 4 + T * (E + 1) * 4)
        w1 = (torch.randn(E, Fe, W, device=dev) / math.sqrt(W)).to(bf)
        w1g = (torch.randn(E, 2 * Fe, W, device=dev) / math.sqrt(W)).to(bf)
        w2 = (torch.randn(E, W, Fe, device=dev) / math.sqrt(Fe)).to(bf)

        def experts(w_up, act, renorm):
            s_, a_, o_, c_ = moe_ops.top_k_gating(logits, K, renormalize=renorm, score_function="softmax")
            return fused_ep.grouped_experts_inference(xe, s_, a_, o_, c_, w_up, w2, act, K)
        add("experts: top-k softmax, squared-relu experts, grouped GEMMs, weighted sum", None, phase,
            lambda: experts(w1, lambda t: M.bias_act_rows(t, None, "relu_sq"), True),
            E * 2 * Fe * W * 2 + T * W * 2 * (1 + 2 * K + 1) + T * K * 2 * Fe * 2, 2.0 * T * K * 2 * Fe * W, "bf16")
        add("experts: softmax gating, gated experts, grouped GEMMs, weighted sum",
            "experts: top-k softmax, squared-relu experts, grouped GEMMs, weighted sum", phase,
            lambda: experts(w1g, F.swiglu, False),
            E * 3 * Fe * W * 2 + T * W * 2 * (1 + 2 * K + 1) + T * K * 3 * Fe * 2, 2.0 * T * K * 3 * Fe * W, "bf16")
        lg = torch.randn(n_seq, VOCAB, device=dev)
        add("scale_softcap (logits)", None, phase, lambda: M.scale_softcap_(lg, 0.5, 30.0), n_seq * VOCAB * 8)
    by_name = {(r_["kernel"], r_["phase"]): r_ for r_ in rows}
    for r_ in rows:                      # distance from the roofline relative to the like kernel's
        if r_["like"]:
            mine = by_name[(r_["like"], r_["phase"])]
            mine["like_of_roofline"] = r_["of_roofline"]
            mine["like_kernel"] = r_["kernel"]
    return rows


# ------------------------------------------------------------------------------------------------ Pifazen beside Kekopel
PIFAZEN = dict(taps=4, rank=64, experts=8, identity=2, groups=2, keep=1, top=2, scale=2.0, limit=7.0,
               yarn=dict(factor=8.0, original=1024, fast=32.0, slow=1.0))


def pifazen_config(z: Dict) -> Dict:
    kinds = ["latent_attention", "channel_delta", "latent_attention_2"]
    lat = {"dim": z["head"], "heads": z["heads"], "kv_rank": LATENT["kv_rank"], "q_rank": LATENT["q_rank"],
           "rot": {"base": 10000.0, "dims": LATENT["rot"]}, "rot_dim": LATENT["rot"],
           "scale": (z["head"] + LATENT["rot"]) ** -0.5, "vdim": z["head"]}
    lat2 = {k: v for k, v in lat.items() if k != "q_rank"}
    lat2["rot"] = {"base": 10000.0, "dims": LATENT["rot"], "scaling": dict(PIFAZEN["yarn"])}
    mixers = {"latent_attention": lat, "latent_attention_2": lat2,
              "channel_delta": {"conv": PIFAZEN["taps"], "dim": z["head"], "heads": z["heads"], "kv_heads": z["heads"],
                                "vdim": z["head"]}}
    mlps = [{"ff": z["ff"], "kind": "dense"},
            {"expert": {"ff": z["ff"] // 4, "limit": PIFAZEN["limit"]}, "kind": "moe",
             "router": {"experts": PIFAZEN["experts"], "identity": PIFAZEN["identity"], "top": PIFAZEN["top"],
                        "groups": {"count": PIFAZEN["groups"], "keep": PIFAZEN["keep"]}, "scale": PIFAZEN["scale"]}}]
    layers = [{"type": kinds[i % 3], "mixer": mixers[kinds[i % 3]], "mlp": mlps[i % 2]} for i in range(z["layers"])]
    return {"architecture": "Pifazen", "layers": layers, "norm": {"eps": 1e-5}, "vocab": VOCAB, "width": z["width"]}


def pifazen_weights(cfg: Dict, device) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(0)
    W, bf = cfg["width"], torch.bfloat16

    def mat(o, i):
        return (torch.randn(o, i, generator=g, device=device) / math.sqrt(i)).to(bf)

    def vec(n, lo=0.5, hi=1.5):
        return (torch.rand(n, generator=g, device=device) * (hi - lo) + lo).to(bf)

    out = {"embed": mat(cfg["vocab"], W), "final.norm": vec(W, -0.2, 0.2)}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        for n in ("1", "2"):
            out[p + "norm" + n], out[p + "ls" + n] = vec(W, -0.2, 0.2), vec(W, 0.2, 0.8)
        if L["type"] == "channel_delta":
            H, G, d, dv, taps, rk = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], PIFAZEN["rank"]
            for n, o in (("q", G * d), ("k", G * d), ("v", H * dv)):
                out[p + "mix." + n], out[p + "mix." + n + ".conv"] = mat(o, W), vec(o * taps, -0.5, 0.5).view(o, taps)
            out[p + "mix.b"], out[p + "mix.A_log"] = mat(H, W), vec(H, -3.0, -1.0)
            out[p + "mix.a1"], out[p + "mix.a2"], out[p + "mix.dt_bias"] = mat(rk, W), mat(H * d, rk), vec(H * d, -1, 1)
            out[p + "mix.g1"], out[p + "mix.g2"] = mat(rk, W), mat(H * dv, rk)
            out[p + "mix.norm"], out[p + "mix.o"] = vec(dv), mat(W, H * dv)
        else:
            H, d, rot, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            if L["type"] == "latent_attention":
                qr = m["q_rank"]
                out[p + "mix.dq"], out[p + "mix.dq.norm"], out[p + "mix.uq"] = mat(qr, W), vec(qr), mat(H * (d + rot), qr)
                out[p + "mix.g"] = mat(H * dv, W)
            else:
                out[p + "mix.q"], out[p + "mix.g"] = mat(H * (d + rot), W), mat(H, W)
            out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = mat(r + rot, W), vec(r)
            out[p + "mix.uk"], out[p + "mix.uv"], out[p + "mix.o"] = mat(H * d, r), mat(H * dv, r), mat(W, H * dv)
        mlp = L["mlp"]
        if mlp["kind"] == "dense":
            out[p + "mlp.up"], out[p + "mlp.up.b"] = mat(mlp["ff"], W), vec(mlp["ff"], -0.1, 0.1)
            out[p + "mlp.down"], out[p + "mlp.down.b"] = mat(W, mlp["ff"]), vec(W, -0.1, 0.1)
            out[p + "mlp.act"] = torch.tensor([0.6, 0.3, 0.2, 0.05], device=device).to(bf)
        else:
            F_, E, n_id = mlp["expert"]["ff"], mlp["router"]["experts"], mlp["router"]["identity"]
            out[p + "mlp.router"], out[p + "mlp.correction"] = mat(E + n_id, W), vec(E + n_id, -0.05, 0.05)
            for e in range(E):
                out[p + f"mlp.e{e}.gate"], out[p + f"mlp.e{e}.up"] = mat(F_, W), mat(F_, W)
                out[p + f"mlp.e{e}.down"] = mat(W, F_)
    return out


def build_pifazen(z: Dict, max_tokens: int, max_seqs: int, pages: int):
    cfg = pifazen_config(z)
    return build_engine_from_state_dict(cfg, pifazen_weights(cfg, "cuda"), _engine_config(max_tokens, max_seqs, pages),
                                        dtype=torch.bfloat16)


def pifazen_kernel_table(z: Dict, prefill: int, batch: int, context: int, timer, hbm_gbs: float,
                         peak_tflops: Dict[str, float]) -> List[Dict]:
    """Every kernel the Pifazen stack adds or takes in a new form, beside the kernel of the Kekopel / Fomalix stacks that
    does the like job (``like``), at prefill (one request) and decode (``batch`` requests) shapes: device time,
    algorithmic bytes and FLOPs, fraction of the roofline (the larger of bytes / copy bandwidth and FLOPs / the peak of
    the unit the products run on)."""
    from ...moe import fused_ep
    from ...ops import functional as F
    from ...ops import moe_ops
    from .kernels import mixer_ops as M
    from .modules.configs import RotaryScalingConfig
    from .modules.implementations import DSLatentSinkAttention
    from .ragged.ragged_wrapper import RaggedBatchWrapper
    dev, bf = "cuda", torch.bfloat16
    W, H, d, ff = z["width"], z["heads"], z["head"], z["ff"]
    r, rot, rk = LATENT["kv_rank"], LATENT["rot"], PIFAZEN["rank"]
    rows: List[Dict] = []

    def add(name, like, phase, fn, nbytes, flops=0.0, pipe=None):
        ms = timer(fn, 5, 3)
        ideal_ms = nbytes / hbm_gbs / 1e6
        if pipe is not None:
            ideal_ms = max(ideal_ms, flops / peak_tflops[pipe] / 1e9)
        rows.append({"kernel": name, "like": like, "phase": phase, "ms": round(ms, 4),
                     "GB_s": round(nbytes / ms / 1e6, 1), "GFLOP_s": round(flops / ms / 1e6, 1), "pipe": pipe or "memory",
                     "of_roofline": round(ideal_ms / ms, 3)})

    for phase, T, n_seq, seen in (("prefill", prefill, 1, 0), ("decode", batch, batch, context)):
        per = T // n_seq
        tot = seen + per
        n_pages_seq = (tot + 63) // 64
        t2s = torch.arange(n_seq, device=dev, dtype=torch.int32).repeat_interleave(per)
        pos = (torch.arange(per, device=dev, dtype=torch.int32) + seen).repeat(n_seq)
        tables = torch.arange(n_seq * n_pages_seq, device=dev, dtype=torch.int32).view(n_seq, n_pages_seq)
        info = torch.tensor([[i * per, per, seen, i] for i in range(n_seq)], dtype=torch.int32, device=dev)
        x32 = torch.randn(T, W, device=dev)
        y = torch.randn(T, W, device=dev).to(bf)
        wv = torch.ones(W, device=dev, dtype=bf)
        # closing a sublayer with a channel scale and opening the next with weights stored around zero
        add("resid_norm_step (channel scale, weight offset)", None, phase,
            lambda: M.resid_norm_step(x32, y, None, None, wv, 1e-5, bf, 1.0, False, wv, 1.0), T * W * (4 + 4 + 2 + 2))
        add("resid_norm_step (multiplier)", "resid_norm_step (channel scale, weight offset)", phase,
            lambda: M.resid_norm_step(x32, y, None, None, wv, 1e-5, bf, 0.5), T * W * (4 + 4 + 2 + 2))
        # latent attention: rotation with scaled frequencies and amplitude, causal attention, output gates
        q = torch.randn(T, H * (d + rot), device=dev).to(bf)
        q_abs = torch.randn(H, T, r, device=dev).to(bf).transpose(0, 1)
        kvp = torch.randn(T, r + rot, device=dev).to(bf)
        kn = torch.ones(r, device=dev, dtype=bf)
        inv, amp = DSLatentSinkAttention.rotary_table(rot, 10000.0, RotaryScalingConfig(**PIFAZEN["yarn"]))
        inv = inv.to(dev)
        inv0 = DSLatentSinkAttention.rotary_table(rot, 10000.0)[0].to(dev)
        cache = torch.randn(n_seq * n_pages_seq, 64, 1, r + rot, device=dev).to(bf)
        prep_bytes = T * ((r + rot) * 4 + H * (r + rot) * (2 + 4))
        add("latent_qk_prepare (scaled frequencies, amplitude)", None, phase,
            lambda: M.latent_qk_prepare(q, q_abs, kvp, kn, inv, cache, t2s, pos, tables, H, d, rot, 1e-5, amp), prep_bytes)
        add("latent_qk_prepare", "latent_qk_prepare (scaled frequencies, amplitude)", phase,
            lambda: M.latent_qk_prepare(q, q_abs, kvp, kn, inv0, cache, t2s, pos, tables, H, d, rot, 1e-5), prep_bytes)
        wrap = RaggedBatchWrapper(max(T, 64), n_seq, n_pages_seq, device=dev)

        class _Seq:
            def __init__(self, i):
                self.seen_tokens, self._b = seen, tables[i].cpu()

            def kv_blocks(self):
                return self._b
        for i in range(n_seq):
            wrap.insert_sequence(_Seq(i), torch.zeros(per, dtype=torch.int32), do_checks=False)
        wrap.finalize()
        atoms, n_long = wrap.atoms(), wrap.atoms_longer_than(M.SHORT_ATOM)
        sink = torch.zeros(H, device=dev)
        ql = torch.randn(T, H, r + rot, device=dev)
        keys_per_q = (per + 1) / 2 if phase == "prefill" else tot
        att_bytes = n_seq * tot * (r + rot) * 2 + T * H * ((r + rot) * 4 + r * 2)
        att_flops = 2.0 * T * H * (2 * r + rot) * keys_per_q
        add("sink_attention, latent rows (causal, no sink)", None, phase,
            lambda: M.sink_attention(ql, cache, None, None, t2s, pos, tables, 0.06, 0, bf, atoms, n_long, value_cols=r),
            att_bytes, att_flops, "fp32")
        add(f"sink_attention, latent rows (window {tot}, sink)", "sink_attention, latent rows (causal, no sink)", phase,
            lambda: M.sink_attention(ql, cache, None, sink, t2s, pos, tables, 0.06, 0, bf, atoms, n_long, window=tot,
                                     value_cols=r), att_bytes, att_flops, "fp32")
        ctx = torch.randn(T, H * d, device=dev).to(bf)
        gpc, gph = torch.randn(T, H * d, device=dev).to(bf), torch.randn(T, (H + 7) // 8 * 8, device=dev).to(bf)
        add("sigmoid_gate_rows (per channel)", None, phase, lambda: M.sigmoid_gate_rows_(ctx, gpc, 1), T * H * d * 6)
        add("sigmoid_gate_rows (per head)", None, phase, lambda: M.sigmoid_gate_rows_(ctx, gph[:, :H], d), T * H * d * 4)
        acc, gl = torch.randn(T, H * d, device=dev).to(bf), torch.randn(T, device=dev)
        add("row_gate_add", "sigmoid_gate_rows (per channel)", phase, lambda: M.row_gate_add_(acc, ctx, gl), T * H * d * 6)
        # delta rule: decay per key channel beside one decay per head
        a_raw, b_raw = torch.randn(T, H * d, device=dev).to(bf), torch.randn(T, (H + 7) // 8 * 8, device=dev).to(bf)
        A_log, dtb, dtb1 = torch.zeros(H, device=dev), torch.zeros(H * d, device=dev), torch.zeros(H, device=dev)
        add("channel_decay_gates", None, phase,
            lambda: M.channel_decay_gates(a_raw, b_raw[:, :H], A_log, dtb, H, d), T * H * d * (2 + 4) + T * H * 6)
        add("recurrence_gates", "channel_decay_gates", phase,
            lambda: M.recurrence_gates(b_raw[:, :H], b_raw[:, :H], A_log, dtb1, "delta"), T * H * (2 * 2 + 2 * 4))
        xs = torch.randn(T, 3 * H * d, device=dev)
        xs[:, : 2 * H * d] /= math.sqrt(d)
        decay_c = torch.rand(T, H * d, device=dev) * 0.1 + 0.9
        decay_h, beta = torch.rand(T, H, device=dev) * 0.1 + 0.9, torch.rand(T, H, device=dev)
        S0 = torch.zeros(n_seq, H, d, d, device=dev)
        sb = (2 if seen else 1) * 4
        rec_flops = 6.0 * T * H * d * d
        add("linear_recurrence (delta, decay per key channel)", None, phase,
            lambda: M.linear_recurrence(xs[:, H * d: 2 * H * d], xs[:, : H * d], xs[:, 2 * H * d:], decay_c, beta, None, S0,
                                        info, H, H, d, d, True),
            n_seq * H * d * d * sb + T * (4 * H * d * 4 + H * d * 4), rec_flops + 2.0 * T * H * d * d, "fp32")
        add("linear_recurrence (delta, decay per head)", "linear_recurrence (delta, decay per key channel)", phase,
            lambda: M.linear_recurrence(xs[:, H * d: 2 * H * d], xs[:, : H * d], xs[:, 2 * H * d:], decay_h, beta, None, S0,
                                        info, H, H, d, d, True),
            n_seq * H * d * d * sb + T * (3 * H * d * 4 + H * d * 4), rec_flops, "fp32")
        o0 = torch.randn(T, H * d, device=dev)
        gate = torch.randn(T, H * d, device=dev).to(bf)
        nw = torch.ones(d, device=dev, dtype=bf)
        add("group_norm_gate (sigmoid gate)", None, phase,
            lambda: M.group_norm_gate(o0, gate, nw, d, 1e-5, False, bf, sigmoid=True), T * H * d * (4 + 2 + 2))
        add("group_norm_gate (silu gate)", "group_norm_gate (sigmoid gate)", phase,
            lambda: M.group_norm_gate(o0, gate, nw, d, 1e-5, False, bf), T * H * d * (4 + 2 + 2))
        # feed-forwards
        hu = torch.randn(T, ff, device=dev).to(bf)
        bu = torch.zeros(ff, device=dev, dtype=bf)
        coef = torch.tensor([0.6, 0.3, 0.2, 0.05], device=dev)
        add("power_norm_act", None, phase, lambda: M.power_norm_act(hu, bu, coef, 1e-5), T * ff * 4)
        add("bias_act_rows (squared relu)", "power_norm_act", phase, lambda: M.bias_act_rows(hu, bu, "relu_sq"), T * ff * 4)
        E, n_id, K, Fe = PIFAZEN["experts"], PIFAZEN["identity"], PIFAZEN["top"], ff // 4
        hg = torch.randn(T * K, 2 * Fe, device=dev).to(bf)
        add("gated_act_rows (clamped)", None, phase, lambda: M.gated_act_rows(hg, "clamped_swish", 7.0), T * K * Fe * 6)
        add("gated_act (silu)", "gated_act_rows (clamped)", phase, lambda: F.gated_act(hg, "silu"), T * K * Fe * 6)
        logits = torch.randn(T, E + n_id, device=dev)
        corr = torch.zeros(E + n_id, device=dev)
        gate_bytes = T * ((E + n_id) * 4 + K * 12)
        add("grouped_top_k_gating (correction, groups, scale)", None, phase,
            lambda: moe_ops.top_k_gating(logits, K, correction=corr, n_groups=PIFAZEN["groups"],
                                         keep_groups=PIFAZEN["keep"], scale=PIFAZEN["scale"]), gate_bytes)
        add("top_k_gating (softmax)", "grouped_top_k_gating (correction, groups, scale)", phase,
            lambda: moe_ops.top_k_gating(logits[:, :E].contiguous(), K, renormalize=True), T * (E * 4 + K * 12))
        xe = torch.randn(T, W, device=dev).to(bf)
        w1 = (torch.randn(E, 2 * Fe, W, device=dev) / math.sqrt(W)).to(bf)
        w2 = (torch.randn(E, W, Fe, device=dev) / math.sqrt(Fe)).to(bf)
        moe_bytes = E * 3 * Fe * W * 2 + T * W * 2 * (1 + 2 * K + 1) + T * K * 3 * Fe * 2
        moe_flops = 2.0 * T * K * 3 * Fe * W

        def experts(identity):
            if identity:
                s, a, o, c = moe_ops.top_k_gating(logits, K, correction=corr, n_groups=PIFAZEN["groups"],
                                                  keep_groups=PIFAZEN["keep"], scale=PIFAZEN["scale"])
                return fused_ep.grouped_experts_inference(xe, s, a, o, c, w1, w2,
                                                          lambda t: M.gated_act_rows(t, "clamped_swish", 7.0), K,
                                                          n_identity=n_id)
            s, a, o, c = moe_ops.top_k_gating(logits[:, :E].contiguous(), K, renormalize=False)
            return fused_ep.grouped_experts_inference(xe, s, a, o, c, w1, w2, F.swiglu, K)
        add("experts: group-limited gating, clamped experts, identity rows copied", None, phase,
            lambda: experts(True), moe_bytes, moe_flops, "bf16")
        add("experts: softmax gating, rows in, grouped GEMMs, weighted sum", "experts: group-limited gating, clamped "
            "experts, identity rows copied", phase, lambda: experts(False), moe_bytes, moe_flops, "bf16")
    by_name = {(r_["kernel"], r_["phase"]): r_ for r_ in rows}
    for r_ in rows:                      # distance from the roofline relative to the like kernel's
        if r_["like"]:
            mine = by_name[(r_["like"], r_["phase"])]
            mine["like_of_roofline"] = r_["of_roofline"]
            mine["like_kernel"] = r_["kernel"]
    return rows


def run(sizes: List[str], prefill: int, batch: int, context: int, steps: int, warmup: int, kernels: bool = True,
        chunk: int = 0, model: str = "fomalix") -> Dict:
    global CHUNK, WINDOW
    if chunk > 0:
        CHUNK = WINDOW = chunk
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            peaks = json.load(f)
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    sm_mhz = float(peaks.get("sm_max_mhz", 1965.0))
    # fp32 FMA lanes: 148 SMs x 128 lanes x 2 FLOPs per clock at the maximum SM clock; tensor cores: the measured GEMM
    peak_tflops = {"fp32": 148 * 128 * 2 * sm_mhz * 1e6 / 1e12, "bf16": float(peaks.get("bf16_tflops", 1590.0))}
    timer = _Timer()
    out = {"metric": "serving tokens/s, hybrid (Fomalix) vs Llama stack of equal size", "dtype": "bf16",
           "data": "synthetic", "weights": "random", "hbm_gbs_denominator": hbm,
           "denominator_source": "measured" if peaks else "fallback", "l2": "256 MB buffer rewritten between forwards",
           "attention_chunk": CHUNK, "fp32_fma_tflops_nominal": round(peak_tflops["fp32"], 1),
           "bf16_tflops_denominator": peak_tflops["bf16"],
           "sizes": {}}
    if model == "kekopel":
        out["metric"] = "serving tokens/s, Kekopel vs hybrid (Fomalix) stack of equal size"
        out["attention_window"], out["latent"] = WINDOW, LATENT
        CHUNK = WINDOW                   # the Fomalix stack's chunks are as long as the Kekopel stack's window
        out["attention_chunk"] = CHUNK
        for name in sizes:
            z = SIZES[name]
            entry = {"config": z,
                     "kekopel": engine_throughput(build_kekopel, z, prefill, batch, context, steps, warmup, timer),
                     "fomalix": engine_throughput(build_hybrid, z, prefill, batch, context, steps, warmup, timer)}
            if kernels:
                entry["kernels"] = kekopel_kernel_table(z, prefill, batch, context, timer, hbm, peak_tflops)
            out["sizes"][name] = entry
        return out
    if model == "pifazen":
        out["metric"] = "serving tokens/s, Pifazen vs Kekopel stack of equal size"
        out["pifazen"], out["latent"] = PIFAZEN, LATENT
        WINDOW = CHUNK = max(WINDOW, prefill, context + steps + warmup + 8)    # the Kekopel window holds every key: equal work
        out["attention_window"] = out["attention_chunk"] = WINDOW
        for name in sizes:
            z = SIZES[name]
            entry = {"config": z,
                     "pifazen": engine_throughput(build_pifazen, z, prefill, batch, context, steps, warmup, timer),
                     "kekopel": engine_throughput(build_kekopel, z, prefill, batch, context, steps, warmup, timer)}
            if kernels:
                entry["kernels"] = pifazen_kernel_table(z, prefill, batch, context, timer, hbm, peak_tflops)
            out["sizes"][name] = entry
        return out
    if model == "ridazen":
        out["metric"] = "serving tokens/s, Ridazen vs a Fomalix stack of attention layers of equal size"
        out["ridazen"] = RIDAZEN
        for name in sizes:
            z = SIZES[name]
            entry = {"config": z,
                     "ridazen": engine_throughput(build_ridazen, z, prefill, batch, context, steps, warmup, timer),
                     "fomalix_attention": engine_throughput(build_attention_stack, z, prefill, batch, context, steps,
                                                            warmup, timer)}
            if kernels:
                entry["kernels"] = ridazen_kernel_table(z, prefill, batch, context, timer, hbm, peak_tflops)
            out["sizes"][name] = entry
        return out
    for name in sizes:
        z = SIZES[name]
        entry = {"config": z,
                 "fomalix": engine_throughput(build_hybrid, z, prefill, batch, context, steps, warmup, timer),
                 "llama": engine_throughput(build_llama, z, prefill, batch, context, steps, warmup, timer)}
        if kernels:
            entry["kernels"] = kernel_table(z, prefill, batch, context, timer, hbm, peak_tflops)
        out["sizes"][name] = entry
    return out
