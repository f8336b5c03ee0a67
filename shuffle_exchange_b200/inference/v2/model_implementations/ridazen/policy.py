"""Ridazen: a decoder-only stack of pre-norm layers with one residual multiplier (``hybrid_model.py``, block form
``"pre_scaled"``).  ``config.json`` lists every layer with its token mixer, the mixer's sizes and its feed-forward, and
may name a span of layers (``loop``) that runs several times with the same weights.

Mixer ``attention``: q | k | v through a short causal filter over time (``conv`` taps, carried per sequence), RMS norm of
every q and k head with one weight each, a query temperature that grows with the logarithm of the position, a learned
bias per head and distance bucket on the scaled scores (no rotation), causal softmax, a sigmoid output gate.
Feed-forward ``moe``: squared-ReLU experts chosen by the largest router logits (with a bias), weighted by the softmax
over the chosen logits, plus a shared expert scaled by a sigmoid per token.  Behind the feed-forward every layer adds a
per-layer token input: its own channels of a second embedding row of the token, gated by a GELU of a projection of the
stream, projected back and RMS-normed.  Final norm, head, logit scale and soft cap.

Checkpoint names: ``embed``, ``side.embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1|norm2``, ``l<i>.mix.*``
(``q``, ``k``, ``v`` with ``.conv`` filters and ``q.norm`` / ``k.norm``, ``rel`` ``[buckets, heads]``, ``g``, ``o``),
``l<i>.mlp.*`` (``router``, ``router.b``, ``e<j>.up|down``, ``shared.up|down|sg``) and ``l<i>.side.gate|proj|norm``.
Linear weights are ``[out, in]``.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ...modules.implementations import DSFilteredBiasAttention
from ..fomalix.policy import _cfg_dict
from ..hybrid_model import DSHybridModel, HybridLayerSpec, HybridSpec, pad_rows
from ..inference_policy_base import InferenceV2Policy
from ..inference_transformer_base import LayerWeights


def pad_cols(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """Zero input columns up to a multiple of 8: the partner of :func:`pad_rows` on the product that follows."""
    extra = (-w.shape[-1]) % multiple
    if extra == 0:
        return w.contiguous()
    return torch.cat([w, w.new_zeros(*w.shape[:-1], extra)], dim=-1).contiguous()


class RidazenPolicy(InferenceV2Policy):

    def spec(self, model_config) -> HybridSpec:
        cfg = _cfg_dict(model_config)
        layers = []
        for L in cfg["layers"]:
            m, kind = L["mixer"], L["type"]
            mlp = L.get("mlp")
            ff: Dict[str, Any] = {}
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ValueError(f"Unsupported feed-forward kind {mlp.get('kind')!r}")
                shared = mlp.get("shared") or {}
                ff = dict(ff_dim=int(mlp["expert"]["ff"]), ff_kind="moe", ff_activation="relu_sq", ff_gated=False,
                          n_experts=int(mlp["router"]["experts"]), top_k=int(mlp["router"]["top"]),
                          moe_score="softmax", moe_renormalize=True, router_bias=True,
                          shared_ff_dim=int(shared.get("ff", 0)))
            if kind != "attention":
                raise ValueError(f"Unknown mixer type {kind!r}")
            temp = m.get("q_temp") or {}
            layers.append(HybridLayerSpec(
                kind="attention", n_heads=int(m["heads"]), n_heads_kv=int(m.get("kv_heads", m["heads"])),
                key_dim=int(m["dim"]), value_dim=int(m.get("vdim", m["dim"])), attn_scale=float(m["scale"]),
                conv_taps=int(m.get("conv", 1)), qk_norm_weight=True, q_temp_coef=float(temp.get("coef", 0.0)),
                q_temp_every=int(temp.get("every", 1)), dist_rows=-1, dist_far=int(m.get("bias_max", 0)),
                out_gate=True, **ff))
        loop = cfg.get("loop") or {}
        side = cfg.get("token_side") or {}
        dt = getattr(model_config, "torch_dtype", None)
        return HybridSpec(vocab_size=int(cfg["vocab"]), model_dim=int(cfg["width"]), layers=layers,
                          norm_eps=float(cfg["norm"]["eps"]), sinusoid_base=None, block_form="pre_scaled",
                          residual_mult=float(cfg.get("residual_mult", 1.0)), token_side_dim=int(side.get("dim", 0)),
                          logit_scale=float(cfg.get("logit_scale", 1.0)),
                          logit_softcap=float(cfg.get("logit_softcap") or 0.0),
                          loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)),
                          loop_times=int(loop.get("times", 1)),
                          dtype=dt if dt in (torch.bfloat16, torch.float32) else torch.bfloat16)

    def resolved_spec(self) -> HybridSpec:
        """The number of distance buckets is the row count of every layer's ``rel`` table, not a configuration entry."""
        spec = super().resolved_spec()
        if getattr(self, "_rel_rows", None) is None:
            self._rel_rows = {name: int(t.shape[0]) for name, t in self._checkpoint_engine.parameters()
                              if name.endswith(".mix.rel")}
        for i, L in enumerate(spec.layers):
            L.dist_rows = self._rel_rows.get(f"l{i}.mix.rel", 0)
        return spec

    # ------------------------------------------------------------------------------------------ weights
    def load_weights(self) -> Dict:
        if self._weights is not None:
            return self._weights
        spec = self.resolved_spec()
        dev, dt = self._device(), spec.dtype
        raw = {name: t.detach() for name, t in self._checkpoint_engine.parameters()}
        used = set()

        def get(name, dtype=dt):
            used.add(name)
            return raw[name].to(dev, dtype).contiguous()

        def cat(names, dtype=dt):
            return torch.cat([get(n, dtype) for n in names], dim=0)

        f32 = torch.float32
        weights: Dict[str, Any] = {"embed": get("embed"), "final_norm_w": get("final.norm"),
                                   "unembed": pad_rows(get("head")), "layers": []}
        if spec.token_side_dim > 0:
            weights["side_embed"] = get("side.embed")
        for i, L in enumerate(spec.layers):
            p, lw = f"l{i}.", LayerWeights()
            m = p + "mix."
            lw["norm1"] = get(p + "norm1")
            lw["w_in"] = pad_rows(cat([m + "q", m + "k", m + "v", m + "g"]))
            # a filter of one tap is a scale per channel: it is applied whenever the checkpoint has the tensors
            has_filter = L.conv_taps > 1 or (m + "q.conv") in raw
            lw["conv_w"] = cat([m + "q.conv", m + "k.conv", m + "v.conv"]) if has_filter else None
            if has_filter and lw["conv_w"].shape[1] != L.conv_taps:
                raise ValueError(f"{m}*.conv have {lw['conv_w'].shape[1]} taps, the configuration says {L.conv_taps}")
            lw["q_norm"], lw["k_norm"] = get(m + "q.norm"), get(m + "k.norm")
            lw["dist_bias"] = (DSFilteredBiasAttention.expand_distance_bias(get(m + "rel", f32), L.dist_far)
                               if L.dist_rows > 0 else None)
            lw["wo"] = get(m + "o")
            if L.ff_dim > 0:
                f = p + "mlp."
                lw["norm2"] = get(p + "norm2")
                gate, bias = [get(f + "router", f32)], [get(f + "router.b", f32)]
                if L.shared_ff_dim > 0:
                    gate.append(get(f + "shared.sg", f32).reshape(1, -1))
                    bias.append(torch.zeros(1, dtype=f32, device=dev))
                    lw["shared_up"] = pad_rows(get(f + "shared.up"))
                    lw["shared_down"] = pad_cols(get(f + "shared.down"))
                lw["moe_gate"], lw["moe_gate_b"] = torch.cat(gate).contiguous(), torch.cat(bias).contiguous()
                lw["moe_w1"] = torch.stack([pad_rows(get(f"{f}e{e}.up")) for e in range(L.n_experts)]).contiguous()
                lw["moe_w2"] = torch.stack([pad_cols(get(f"{f}e{e}.down")) for e in range(L.n_experts)]).contiguous()
            if spec.token_side_dim > 0:
                lw["side_gate"] = pad_rows(get(p + "side.gate"))
                lw["side_proj"] = pad_cols(get(p + "side.proj"))
                lw["side_norm"] = get(p + "side.norm")
            weights["layers"].append(lw)
        self.container_map.set_unmapped_params([n for n in raw if n not in used])
        self._weights = weights
        return weights

    def build_model(self, engine_config, mp_group=None, state_manager=None) -> DSHybridModel:
        self._engine_config = engine_config
        if mp_group is not None:
            self._mp_group = mp_group
        spec = self.resolved_spec()
        model = DSHybridModel(spec, self.load_weights(), engine_config, state_manager, self._mp_group)
        model.model_config = self._model_config
        return model
