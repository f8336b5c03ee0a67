"""Pifazen: a decoder-only stack of pre-norm layers with a learned scale per layer, sublayer and channel
(``hybrid_model.py``, block form ``"pre_scaled"`` with ``layer_scale``): ``x += ls1 (.) mixer(n1(x))``, ``x += ls2 (.)
ff(n2(x))`` where ``n(x) = x / rms(x) * (1 + w)`` (the norm weights are stored around zero).  ``config.json`` lists every
layer with its token mixer, the mixer's sizes and its feed-forward; a layer with ``weights_of: j`` has no tensors of
its own and runs with layer ``j``'s, on its own cache or state.  The embedding table is also the head.

Mixers.  ``channel_delta``: gated delta rule with a separate decay for every key channel of every head (``channel_delta_mixer``): q | k | v
through a short causal convolution and SiLU, q and k unit vectors, write strength ``sigmoid(W_b h)``, decay
``exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias))``, per-head RMS norm times ``sigmoid(W_g2 W_g1 h)``.
``latent_attention``: queries through a normalised latent, keys and values as up-projections of one normalised latent
per token plus a single rotated key slice that every head uses (interleaved pairs), causal softmax, one sigmoid gate per output
channel.  ``latent_attention_2``: queries straight from the input, rotation frequencies slowed by wavelength
(the four numbers under ``rot.scaling``) with scaled cos and sin, one sigmoid gate per head.

Feed-forwards.  ``dense``: ``W_down act(W_up h + b) + b`` with the three-power normalised activation ``a N(z) + b N(z^2) +
c N(z^3) + e``.  ``moe``: clamped gated experts without biases (``a = min(gate, L)``, ``b = max(-L, min(up, L))``,
``a sigmoid(1.702 a) (1 + b)``); softmax scores over ``experts + identity`` router outputs, the choice made by score +
``correction`` inside the best ``groups.keep`` of ``groups.count`` contiguous blocks, weights = chosen scores / their
sum, times the router's ``scale``; the router's trailing ``identity`` outputs stand for experts that hand their input on.

Checkpoint names: ``embed``, ``final.norm``, and per layer ``l<i>.norm1|norm2|ls1|ls2``, ``l<i>.mix.*`` (channel_delta:
``q``, ``k``, ``v`` with ``.conv`` filters, ``b``, ``A_log``, ``a1``, ``a2``, ``dt_bias``, ``g1``, ``g2``, ``norm``, ``o``;
latent attention: ``dq``, ``dq.norm``, ``uq`` or ``q``, ``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``g``, ``o``) and
``l<i>.mlp.*`` (dense: ``up``, ``up.b``, ``down``, ``down.b``, ``act``; experts: ``router``, ``correction``,
``e<j>.gate|up|down``).  Linear weights are ``[out, in]``.
"""
from __future__ import annotations

from typing import Any, Dict, List

import torch

from ..fomalix.policy import _cfg_dict
from ..hybrid_model import DSHybridModel, HybridLayerSpec, HybridSpec, pad_rows
from ..inference_policy_base import InferenceV2Policy
from ..inference_transformer_base import LayerWeights
from ..ridazen.policy import pad_cols


def weight_owner(layers: List[Dict], i: int) -> int:
    """Index of the layer whose tensors layer ``i`` runs with (``weights_of`` may point at a layer that borrows too)."""
    seen = set()
    while layers[i].get("weights_of") is not None:
        if i in seen:
            raise ValueError(f"layer {i}: weights_of forms a cycle")
        seen.add(i)
        i = int(layers[i]["weights_of"])
        if not 0 <= i < len(layers):
            raise ValueError(f"weights_of names layer {i}, the stack has {len(layers)}")
    return i


class PifazenPolicy(InferenceV2Policy):

    def spec(self, model_config) -> HybridSpec:
        cfg = _cfg_dict(model_config)
        layers = []
        for L in cfg["layers"]:
            m, kind = L["mixer"], L["type"]
            mlp = L.get("mlp")
            ff: Dict[str, Any] = {}
            if mlp is not None:
                if mlp["kind"] == "dense":
                    ff = dict(ff_dim=int(mlp["ff"]), ff_kind="biased", ff_activation="power_norm")
                elif mlp["kind"] == "moe":
                    r = mlp["router"]
                    groups = r.get("groups") or {}
                    ff = dict(ff_dim=int(mlp["expert"]["ff"]), ff_kind="moe", ff_activation="clamped_swish",
                              ff_limit=float(mlp["expert"]["limit"]), n_experts=int(r["experts"]), top_k=int(r["top"]),
                              moe_score="softmax", moe_correction=True, moe_groups=int(groups.get("count", 1)),
                              moe_keep_groups=int(groups.get("keep", groups.get("count", 1))),
                              moe_scale=float(r.get("scale", 1.0)), moe_identity=int(r.get("identity", 0)))
                else:
                    raise ValueError(f"Unsupported feed-forward kind {mlp['kind']!r}")
            if kind in ("latent_attention", "latent_attention_2"):
                rot = m.get("rot") or {}
                sc = rot.get("scaling")
                direct = kind == "latent_attention_2"
                layers.append(HybridLayerSpec(
                    kind="latent_attention", n_heads=int(m["heads"]), n_heads_kv=1, key_dim=int(m["dim"]),
                    value_dim=int(m["vdim"]), attn_scale=float(m["scale"]), sink=False,
                    q_rank=0 if direct else int(m["q_rank"]), kv_rank=int(m["kv_rank"]), rot_dim=int(m["rot_dim"]),
                    rot_dims=int(rot.get("dims", m["rot_dim"])), rot_base=float(rot.get("base", 10000.0)),
                    rot_scaling=None if not sc else (float(sc["factor"]), float(sc["original"]), float(sc["fast"]),
                                                     float(sc["slow"])),
                    out_gate=True, gate_per_head=direct, q_direct=direct, **ff))
            elif kind == "channel_delta":
                layers.append(HybridLayerSpec(
                    kind="channel_delta", n_heads=int(m["heads"]), n_heads_kv=int(m.get("kv_heads", m["heads"])),
                    key_dim=int(m["dim"]), value_dim=int(m["vdim"]), conv_taps=int(m.get("conv", 1)), **ff))
            else:
                raise ValueError(f"Unknown mixer type {kind!r}")
        dt = getattr(model_config, "torch_dtype", None)
        return HybridSpec(vocab_size=int(cfg["vocab"]), model_dim=int(cfg["width"]), layers=layers,
                          norm_eps=float(cfg["norm"]["eps"]), sinusoid_base=None, block_form="pre_scaled",
                          layer_scale=True, norm_weight_offset=1.0,
                          dtype=dt if dt in (torch.bfloat16, torch.float32) else torch.bfloat16)

    # ------------------------------------------------------------------------------------------ weights
    def load_weights(self) -> Dict:
        if self._weights is not None:
            return self._weights
        spec = self.resolved_spec()
        cfg_layers = _cfg_dict(self._model_config)["layers"]
        dev, dt = self._device(), spec.dtype
        raw = {name: t.detach() for name, t in self._checkpoint_engine.parameters()}
        used = set()

        def get(name, dtype=dt):
            used.add(name)
            return raw[name].to(dev, dtype).contiguous()

        def cat(names, dtype=dt):
            return torch.cat([get(n, dtype) for n in names], dim=0)

        f32 = torch.float32
        embed = get("embed")
        weights: Dict[str, Any] = {"embed": embed, "final_norm_w": get("final.norm"), "unembed": pad_rows(embed),
                                   "layers": [None] * len(spec.layers)}
        for i, L in enumerate(spec.layers):
            if weight_owner(cfg_layers, i) != i:
                continue
            p, lw = f"l{i}.", LayerWeights()
            m = p + "mix."
            lw["norm1"], lw["ls1"] = get(p + "norm1"), get(p + "ls1")
            if L.kind == "latent_attention":
                H, d, r, dv = L.n_heads, L.key_dim, L.kv_rank, L.value_dim
                lw["w_in"] = pad_rows(cat([m + ("q" if L.q_direct else "dq"), m + "dkv", m + "g"]))
                if not L.q_direct:
                    lw["q_norm"], lw["w_uq"] = get(m + "dq.norm"), pad_rows(get(m + "uq"))
                lw["kv_norm"] = get(m + "dkv.norm")
                lw["w_uk"] = get(m + "uk").view(H, d, r).contiguous()
                lw["w_uv_t"] = get(m + "uv").view(H, dv, r).transpose(1, 2).contiguous()
            else:
                H, n, dv = L.n_heads, L.key_dim, L.value_dim
                # the two-step projections' first steps ride in the fused projection, their widths padded to whole
                # 16-byte rows (zero rows here, zero columns in the second step)
                lw["w_in"] = pad_rows(torch.cat([cat([m + "q", m + "k", m + "v"]), pad_rows(get(m + "b")),
                                                 pad_rows(get(m + "a1")), pad_rows(get(m + "g1"))], dim=0))
                lw["conv_w"] = cat([m + "q.conv", m + "k.conv", m + "v.conv"])
                if lw["conv_w"].shape[1] != L.conv_taps:
                    raise ValueError(f"{m}*.conv have {lw['conv_w'].shape[1]} taps, the configuration says {L.conv_taps}")
                lw["A_log"], lw["dt_bias"] = get(m + "A_log", f32), get(m + "dt_bias", f32)
                lw["w_a2"], lw["w_g2"] = pad_rows(pad_cols(get(m + "a2"))), pad_rows(pad_cols(get(m + "g2")))
                lw["norm"] = get(m + "norm")
            lw["wo"] = get(m + "o")
            if L.ff_dim > 0:
                lw["norm2"], lw["ls2"] = get(p + "norm2"), get(p + "ls2")
                f = p + "mlp."
                if L.ff_kind == "moe":
                    lw["moe_gate"], lw["moe_correction"] = get(f + "router", f32), get(f + "correction", f32)
                    if lw["moe_gate"].shape[0] != L.n_experts + L.moe_identity:
                        raise ValueError(f"{f}router has {lw['moe_gate'].shape[0]} rows for {L.n_experts} experts and "
                                         f"{L.moe_identity} identity experts")
                    lw["moe_w1"] = torch.stack([cat([f"{f}e{e}.gate", f"{f}e{e}.up"]) for e in range(L.n_experts)])
                    lw["moe_w2"] = torch.stack([get(f"{f}e{e}.down") for e in range(L.n_experts)]).contiguous()
                else:
                    lw["w_up"], lw["b_up"] = get(f + "up"), get(f + "up.b")
                    lw["w_down"], lw["b_down"] = get(f + "down"), get(f + "down.b")
                    lw["act_coef"] = get(f + "act", f32)
            weights["layers"][i] = lw
        for i in range(len(spec.layers)):          # borrowed layers: the owner's tensors, not a copy
            weights["layers"][i] = weights["layers"][weight_owner(cfg_layers, i)]
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
