"""Pifazen in the ragged engine against the plain evaluation in ``pifazen_oracle.py`` (float64, whole sequences, no cache):
every mechanism alone, prefill against token-by-token decoding, prompt portions down to two tokens, unequal batches,
reuse of cache pages and state slots, keys and writes far back and at page borders, the first tokens, long decoding,
other sizes, layers that borrow weights, and greedy generation through the scheduler.  Runs on the PyTorch branch of
every op without a GPU; ``test_pifazen_gpu.py`` runs the same cases on the CUDA kernels."""
import copy
import math

import pytest
import torch

import pifazen_oracle as O
from shuffle_exchange_b200.inference.v2.config_v2 import RaggedInferenceEngineConfig
from shuffle_exchange_b200.inference.v2.engine_factory import build_engine_from_state_dict
from shuffle_exchange_b200.inference.v2.inference_utils import ActivationType, DtypeEnum
from shuffle_exchange_b200.inference.v2.kernels import mixer_ops as M
from shuffle_exchange_b200.inference.v2.modules import heuristics
from shuffle_exchange_b200.inference.v2.modules.configs import DSMoEConfig, RotaryScalingConfig
from shuffle_exchange_b200.inference.v2.modules.implementations import DSLatentSinkAttention
from shuffle_exchange_b200.inference.v2.ragged.ragged_manager import DSStateManagerConfig
from shuffle_exchange_b200.inference.v2.scheduler import generate
from shuffle_exchange_b200.ops import moe_ops

DEV = "cuda" if torch.cuda.is_available() else "cpu"

MOE = {"expert": {"ff": 16, "limit": 1.5}, "kind": "moe",
       "router": {"experts": 6, "groups": {"count": 4, "keep": 2}, "identity": 2, "scale": 1.5, "top": 3}}
DENSE = {"ff": 40, "kind": "dense"}
LAT = {"type": "latent_attention",
       "mixer": {"dim": 8, "heads": 3, "kv_rank": 20, "q_rank": 12, "rot": {"base": 1000.0, "dims": 4}, "rot_dim": 4,
                 "scale": 0.3, "vdim": 12},
       "mlp": MOE}
LAT2 = {"type": "latent_attention_2",
        "mixer": {"dim": 4, "heads": 4, "kv_rank": 12,
                  "rot": {"base": 200.0, "dims": 8, "scaling": {"factor": 4.0, "fast": 4.0, "original": 16, "slow": 1.0}},
                  "rot_dim": 8, "scale": 0.4, "vdim": 8},
        "mlp": DENSE}
DELTA = {"type": "channel_delta", "mixer": {"conv": 3, "dim": 8, "heads": 4, "kv_heads": 2, "vdim": 12}, "mlp": MOE}


def make_cfg(layers, width=24, vocab=53, eps=1e-5):
    return {"architecture": "Pifazen", "layers": copy.deepcopy(layers), "norm": {"eps": eps}, "vocab": vocab,
            "width": width}


STACK = make_cfg([LAT2, DELTA, LAT, dict(DELTA, mlp=None), dict(DELTA, weights_of=1), dict(LAT, weights_of=2)])


def make_engine(cfg, W, dtype=torch.float32, blocks=64, block_size=4, max_live=4, max_tokens=256):
    sm = DSStateManagerConfig(max_tracked_sequences=max_live, max_ragged_sequence_count=max_live,
                              max_ragged_batch_size=max_tokens, max_context=blocks * block_size, num_kv_blocks=blocks)
    return build_engine_from_state_dict(cfg, W, RaggedInferenceEngineConfig(state_manager=sm, kv_block_size=block_size),
                                        dtype=dtype)


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def feed(engine, uid, toks, sizes):
    """Give ``toks`` to the engine in portions of the given sizes (cycled); returns the logits of every token."""
    out, lo, i = [], 0, 0
    while lo < len(toks):
        n = min(sizes[i % len(sizes)], len(toks) - lo)
        i += 1
        out.append(engine.put([uid], [torch.tensor(toks[lo: lo + n])], logit_positions=[list(range(n))]))
        lo += n
    return torch.cat(out).double().cpu()


def close(got, want, tol=2e-4):
    """Difference with the mean over the vocabulary taken off, relative to the spread of the expected logits."""
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    err = d.pow(2).mean(-1).sqrt() / want.std()
    assert err.max() < tol, f"worst row {int(err.argmax())}: {float(err.max()):.3e}"


@pytest.fixture(scope="module")
def stack():
    W = O.random_weights(STACK, seed=4)
    toks = tokens(47, STACK["vocab"], 5)
    return W, toks, O.forward(STACK, W, toks)


# ------------------------------------------------------------------------------------------------ single mechanisms
@pytest.mark.parametrize("dims,base,scaling", [
    (8, 200.0, {"factor": 4.0, "fast": 4.0, "original": 16, "slow": 1.0}),
    (64, 10000.0, {"factor": 40.0, "fast": 32.0, "original": 4096, "slow": 1.0}),
    (32, 5e5, {"factor": 2.0, "fast": 8.0, "original": 300, "slow": 2.0}),
    (6, 50.0, {"factor": 8.0, "fast": 1.0, "original": 6, "slow": 1.0}),        # the ramp's ends coincide
    (16, 1e4, {"factor": 1.0, "fast": 32.0, "original": 64, "slow": 1.0}),      # factor one: nothing changes
    (12, 777.0, None), (0, 10.0, None)])
def test_rotation_frequencies_and_amplitude(dims, base, scaling):
    sc = None if scaling is None else RotaryScalingConfig(**scaling)
    f, amp = DSLatentSinkAttention.rotary_table(dims, base, sc)
    want_f, want_amp = O.rotary_frequencies({"dims": dims, "base": base, "scaling": scaling})
    assert f.dtype == torch.float32 and f.numel() == dims // 2
    assert torch.allclose(f.double(), torch.tensor(want_f, dtype=torch.float64), rtol=1e-7, atol=0)
    assert amp == pytest.approx(want_amp, rel=1e-12)
    if scaling is not None and scaling["factor"] > 1 and dims:
        plain, _ = O.rotary_frequencies({"dims": dims, "base": base})
        ratio = [a / b for a, b in zip(want_f, plain)]
        assert all(x <= y + 1e-12 for x, y in zip(ratio[1:], ratio))          # slower and slower along the pairs
        assert min(ratio) >= 1 / scaling["factor"] - 1e-12 and want_amp > 1


def _rope_and_cache(q, kv, w, freqs, amp, H, d, rot, cuts, block_size=4):
    """Key latent norm, rotation and cache append in portions; returns the rotated query parts and the cached rows."""
    T, r = kv.shape[0], kv.shape[1] - rot
    pages = (T + block_size - 1) // block_size
    cache = torch.full((pages + 1, block_size, 1, r + rot), 9.0, device=DEV)
    tables = torch.arange(pages, 0, -1, dtype=torch.int32, device=DEV).view(1, pages)
    outs, lo = [], 0
    for n in cuts:
        t2s = torch.zeros(n, dtype=torch.int32, device=DEV)
        pos = torch.arange(lo, lo + n, dtype=torch.int32, device=DEV)
        q_abs = torch.zeros(n, H, r, device=DEV)
        outs.append(M.latent_qk_prepare(q[lo: lo + n].to(DEV).contiguous(), q_abs, kv[lo: lo + n].to(DEV).contiguous(),
                                        w.to(DEV), freqs.to(DEV), cache, t2s, pos, tables, H, d, rot, 1e-5, amp).cpu())
        lo += n
    rows = cache.cpu()[tables[0].long().cpu()].reshape(-1, r + rot)[:T]
    return torch.cat(outs).double()[:, :, r:], rows.double()


@pytest.mark.parametrize("H,d,rot,n_rot,r", [(3, 8, 4, 4, 20), (2, 5, 6, 4, 7), (1, 4, 16, 16, 40)])
def test_rotated_parts_carry_the_amplitude_and_positions_count_from_zero(H, d, rot, n_rot, r):
    g = torch.Generator().manual_seed(H)
    T = 19
    q, kv, w = torch.randn(T, H * (d + rot), generator=g), torch.randn(T, r + rot, generator=g), torch.randn(r, generator=g)
    rot_cfg = {"dims": n_rot, "base": 300.0, "scaling": {"factor": 6.0, "fast": 3.0, "original": 12, "slow": 0.5}}
    freqs, amp = DSLatentSinkAttention.rotary_table(n_rot, 300.0, RotaryScalingConfig(**rot_cfg["scaling"]))
    of, oa = O.rotary_frequencies(rot_cfg)
    want_q = O.rotate_pairs(q.double().view(T, H, d + rot)[:, :, d:], of, oa)
    want_k = O.rotate_pairs(kv.double()[:, r:], of, oa)
    want_c = O.rms_norm(kv.double()[:, :r], w.double(), 1e-5)
    for cuts in ([T], [1, 2, 5, 11]):
        got_q, rows = _rope_and_cache(q, kv, w, freqs, amp, H, d, rot, cuts)
        assert torch.allclose(got_q, want_q, atol=2e-5) and torch.allclose(rows[:, r:], want_k, atol=2e-5)
        assert torch.allclose(rows[:, :r], want_c, atol=2e-5)
    assert torch.allclose(want_q[0], oa * q.double().view(T, H, d + rot)[0, :, d:].clone().index_fill_(
        -1, torch.arange(n_rot, rot), 0) + q.double().view(T, H, d + rot)[0, :, d:].clone().index_fill_(
        -1, torch.arange(0, n_rot), 0))                       # position 0: no turn, only the amplitude


def _recurrence(k, q, v, a_raw, b_raw, A_log, dt_bias, H, G, n, dv, cuts, slot=1):
    """Decay per channel and the delta rule in portions, on a state slot another sequence has used."""
    state = torch.full((3, H, dv, n), 5.0, device=DEV)
    outs, lo = [], 0
    for c in cuts:
        info = torch.tensor([[0, c, lo, slot]], dtype=torch.int32, device=DEV)
        decay, beta = M.channel_decay_gates(a_raw[lo: lo + c].to(DEV), b_raw[lo: lo + c].to(DEV), A_log.to(DEV),
                                            dt_bias.to(DEV), H, n)
        outs.append(M.linear_recurrence(k[lo: lo + c].to(DEV).contiguous(), q[lo: lo + c].to(DEV).contiguous(),
                                        v[lo: lo + c].to(DEV).contiguous(), decay, beta, None, state, info, H, G, n, dv,
                                        True).cpu())
        lo += c
    assert torch.all(state[[0, 2]] == 5.0)
    return torch.cat(outs).double()


def _recurrence_oracle(k, q, v, a_raw, b_raw, A_log, dt_bias, H, G, n, dv):
    T = k.shape[0]
    g = torch.exp(-torch.exp(A_log.double())[None, :, None] * O.softplus(a_raw.double() + dt_bias.double()).view(T, H, n))
    beta = torch.sigmoid(b_raw.double())
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for h in range(H):
        S = torch.zeros(n, dv, dtype=torch.float64)
        kh, qh = k.double().view(T, G, n)[:, h // (H // G)], q.double().view(T, G, n)[:, h // (H // G)]
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v.double().view(T, H, dv)[t, h] - S.T @ kh[t])
            S = S + torch.outer(kh[t], u)
            out[t, h] = S.T @ qh[t]
    return out.reshape(T, H * dv)


@pytest.mark.parametrize("H,G,n,dv", [(4, 2, 8, 12), (3, 3, 5, 3), (2, 1, 40, 36), (1, 1, 130, 20), (6, 2, 64, 17)])
def test_delta_rule_with_a_decay_per_key_channel(H, G, n, dv):
    g = torch.Generator().manual_seed(n)
    T = 29
    k, q = torch.randn(T, G * n, generator=g) / math.sqrt(n), torch.randn(T, G * n, generator=g)
    v, a_raw, b_raw = torch.randn(T, H * dv, generator=g), torch.randn(T, H * n, generator=g), torch.randn(T, H, generator=g)
    A_log, dt_bias = torch.randn(H, generator=g), torch.randn(H * n, generator=g)
    want = _recurrence_oracle(k, q, v, a_raw, b_raw, A_log, dt_bias, H, G, n, dv)
    for cuts in ([T], [1, 1, 2, 8, 9, 8], [16, 13]):
        got = _recurrence(k, q, v, a_raw, b_raw, A_log, dt_bias, H, G, n, dv, cuts)
        assert torch.allclose(got, want, atol=3e-5, rtol=1e-4), float((got - want).abs().max())


def test_a_channel_that_does_not_decay_remembers_a_write_hundreds_of_tokens_back():
    """Two key channels: channel 0 keeps its rows of the state (decay ~ 1), channel 1 loses them at once (decay ~ 0).  A
    value written through channel 0 at the first token is read at the last one, the same write through channel 1 is
    gone at the next token; one decay per head could not do both."""
    H = G = 1
    n, dv, T = 2, 4, 300
    k, q, v = torch.zeros(T, n), torch.zeros(T, n), torch.zeros(T, dv)
    a_raw = torch.zeros(T, n)
    a_raw[:, 0], a_raw[:, 1] = -40.0, 40.0                 # softplus: ~0 and 40
    b_raw = torch.full((T, 1), 40.0)                       # write strength one
    k[0] = torch.tensor([1.0, 1.0])
    v[0] = torch.tensor([1.0, 2.0, 3.0, 4.0])
    q[1], q[T - 1] = torch.tensor([0.0, 1.0]), torch.tensor([1.0, 0.0])
    q[2] = torch.tensor([1.0, 1.0])
    for cuts in ([T], [1] * T, [150, 2, 148]):
        got = _recurrence(k, q, v, a_raw, b_raw, torch.zeros(1), torch.zeros(n), H, G, n, dv, cuts)
        assert torch.allclose(got[T - 1], v[0].double(), atol=1e-4)          # through the channel that keeps
        assert got[1].abs().max() < 1e-6                                     # through the channel that forgets
        assert torch.allclose(got[2], v[0].double(), atol=1e-4)
    assert torch.allclose(got, _recurrence_oracle(k, q, v, a_raw, b_raw, torch.zeros(1), torch.zeros(n), H, G, n, dv),
                          atol=1e-5)


@pytest.mark.parametrize("T,F,bias", [(5, 40, True), (3, 7, False), (2, 1024, True), (1, 300, True)])
def test_three_power_normalised_activation(T, F, bias):
    g = torch.Generator().manual_seed(F)
    x = torch.randn(T, F, generator=g) * 3
    b = torch.randn(F, generator=g) if bias else None
    coef = torch.tensor([0.7, -0.4, 0.3, 0.1])
    z = x.double() + (b.double() if bias else 0.0)
    want = O.three_power_norm(z, coef.double(), 1e-5)
    got = M.power_norm_act(x.to(DEV), None if b is None else b.to(DEV), coef.to(DEV), 1e-5)
    assert torch.allclose(got.double().cpu(), want, atol=2e-5, rtol=1e-5)
    # each power is normalised on its own: doubling the input leaves the result unchanged but for eps
    twice = M.power_norm_act((2 * z).float().to(DEV), None, coef.to(DEV), 1e-12)
    once = M.power_norm_act(z.float().to(DEV), None, coef.to(DEV), 1e-12)
    assert torch.allclose(twice, once, atol=1e-4)


@pytest.mark.parametrize("group", [1, 12])
def test_sigmoid_gates_per_channel_and_per_head(group):
    g = torch.Generator().manual_seed(group)
    T, W = 9, 48
    x, wide = torch.randn(T, W, generator=g), torch.randn(T, 100, generator=g)
    gate = wide[:, 8: 8 + W // group]
    want = x.double() * torch.sigmoid(gate.double()).repeat_interleave(group, dim=1)
    got = M.sigmoid_gate_rows_(x.clone().to(DEV), wide.to(DEV)[:, 8: 8 + W // group], group)
    assert torch.allclose(got.double().cpu(), want, atol=1e-6)
    odd = M.sigmoid_gate_rows_(x[:, :45].contiguous().to(DEV), wide.to(DEV)[:, 3: 3 + 45 // (3 if group > 1 else 1)],
                               3 if group > 1 else 1)
    want = x[:, :45].double() * torch.sigmoid(wide[:, 3: 3 + 45 // (3 if group > 1 else 1)].double()).repeat_interleave(
        3 if group > 1 else 1, dim=1)
    assert torch.allclose(odd.double().cpu(), want, atol=1e-6)


def test_residual_step_with_a_channel_scale_and_weights_stored_around_zero():
    g = torch.Generator().manual_seed(11)
    T, W = 7, 20
    x, y = torch.randn(T, W, generator=g), torch.randn(T, W, generator=g)
    ls, w = torch.randn(W, generator=g), torch.randn(W, generator=g) * 0.1
    r = x.clone().to(DEV)
    out = M.resid_norm_step(r, y.to(DEV), None, None, w.to(DEV), 1e-4, torch.float32, 1.0, False, ls.to(DEV), 1.0)
    want = x.double() + ls.double() * y.double()
    assert torch.allclose(r.double().cpu(), want, atol=1e-5)
    assert torch.allclose(out.double().cpu(), O.offset_norm(want, w.double(), 1e-4), atol=1e-5)
    r = x.clone().to(DEV)
    out = M.resid_norm_step(r, None, None, None, w.to(DEV), 1e-4, torch.float32, 1.0, False, None, 1.0)
    assert torch.allclose(out.double().cpu(), O.offset_norm(x.double(), w.double(), 1e-4), atol=1e-5)


def _experts(E, n_id, K, groups, keep, scale, limit, T=23, W=16, Fe=10, seed=0, correction=None):
    g = torch.Generator().manual_seed(seed + E)
    h = torch.randn(T, W, generator=g)
    P = {"router": torch.randn(E + n_id, W, generator=g),
         "correction": torch.randn(E + n_id, generator=g) * 0.3 if correction is None else correction}
    for e in range(E):
        P[f"e{e}.gate"], P[f"e{e}.up"] = torch.randn(Fe, W, generator=g) / 2, torch.randn(Fe, W, generator=g) / 2
        P[f"e{e}.down"] = torch.randn(W, Fe, generator=g) / 4
    mlp = {"router": {"experts": E, "identity": n_id, "top": K, "groups": {"count": groups, "keep": keep}, "scale": scale},
           "expert": {"ff": Fe, "limit": limit}}
    mod = heuristics.instantiate_moe(DSMoEConfig(
        max_tokens=64, model_dim=W, intermediate_features=Fe, n_experts=E, top_k=K, input_dtype=DtypeEnum.fp32,
        output_dtype=DtypeEnum.fp32, activation=ActivationType.CLAMPED_SWIGLU, router_dtype=DtypeEnum.fp32,
        score_correction=True, n_groups=groups, keep_groups=keep, score_scale=scale, identity_experts=n_id,
        activation_limit=limit), None)
    w1 = torch.stack([torch.cat([P[f"e{e}.gate"], P[f"e{e}.up"]]) for e in range(E)])
    w2 = torch.stack([P[f"e{e}.down"] for e in range(E)])
    got = mod(h.to(DEV), P["router"].to(DEV), w1.to(DEV), w2.to(DEV), correction=P["correction"].to(DEV))
    return h, P, mlp, got.double().cpu()


@pytest.mark.parametrize("E,n_id,K,groups,keep,scale,limit", [
    (6, 2, 3, 4, 2, 1.5, 1.5), (4, 0, 2, 1, 1, 1.0, 7.0), (5, 3, 4, 2, 2, 2.5, 0.5), (9, 1, 1, 5, 1, 1.0, 1.0),
    (8, 8, 8, 4, 2, 0.5, 2.0), (3, 0, 3, 3, 3, 1.0, 1.0)])
def test_clamped_experts_chosen_among_groups_with_identity_experts(E, n_id, K, groups, keep, scale, limit):
    h, P, mlp, got = _experts(E, n_id, K, groups, keep, scale, limit)
    want = O.expert_ff(h.double(), {k: v.double() for k, v in P.items()}, mlp)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), float((got - want).abs().max())


def test_the_correction_chooses_but_does_not_weigh_and_closed_groups_lose_to_negative_choices():
    """A correction of +5 on the last expert (an identity expert) puts it into every token's choice, yet its weight is
    its plain score.  Corrections of -3 everywhere but for group 0's -9 make every choice value negative: experts of the
    closed groups must not win with a value of 0."""
    E, n_id, K, groups, keep = 6, 2, 2, 4, 1
    corr = torch.zeros(E + n_id)
    corr[-1] = 5.0
    h, P, mlp, got = _experts(E, n_id, K, groups, keep, 1.0, 1.0, correction=corr, seed=3)
    z = (h @ P["router"].T).float()
    sc, assign, _, _ = moe_ops.top_k_gating(z.to(DEV), K, correction=corr.to(DEV), n_groups=groups, keep_groups=keep)
    assert bool((assign.cpu() >= E).all())                         # the kept group is the last one: both identity experts
    s = torch.softmax(z.double(), -1)
    picked = s.gather(1, assign.cpu().long())
    assert torch.allclose(sc.double().cpu(), picked / picked.sum(-1, keepdim=True), atol=1e-6)
    assert torch.allclose(got, h.double(), atol=1e-5)              # weights sum to one, both experts return the input
    corr = torch.full((E + n_id,), -3.0)
    corr[:2] = -9.0
    h, P, mlp, got = _experts(E, n_id, K, groups, keep, 1.0, 1.0, correction=corr, seed=4)
    want = O.expert_ff(h.double(), {k: v.double() for k, v in P.items()}, mlp)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4)
    z = (h @ P["router"].T).float()
    _, assign, _, counts = moe_ops.top_k_gating(z.to(DEV), K, correction=corr.to(DEV), n_groups=groups, keep_groups=keep)
    a = assign.cpu()
    assert bool((a // 2 == (a // 2)[:, :1]).all()) and bool((a >= 2).all())     # one group per token, never group 0
    assert int(counts.sum()) == a.numel()


@pytest.mark.parametrize("layer", [LAT, LAT2, DELTA, dict(LAT, mlp=None), dict(DELTA, mlp=DENSE),
                                   dict(LAT2, mlp=dict(MOE, router={"experts": 3, "top": 3, "identity": 0}))],
                         ids=["latent_experts", "direct_queries_dense", "delta_experts", "mixer_alone", "delta_dense",
                              "all_experts_no_groups"])
def test_one_layer_of_each_kind(layer):
    cfg = make_cfg([layer])
    W = O.random_weights(cfg, seed=1)
    toks = tokens(23, cfg["vocab"], 2)
    want = O.forward(cfg, W, toks)
    eng = make_engine(cfg, W)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [3, 1, 2]), want)


def test_stream_after_every_layer(stack):
    W, toks, _ = stack
    handed = []
    O.forward(STACK, W, toks, handed)
    eng = make_engine(STACK, W)
    eng.model().layer_outputs = []
    feed(eng, 1, toks, [len(toks)])
    assert len(handed) == len(eng.model().layer_outputs) == len(STACK["layers"])
    for got, want in zip(eng.model().layer_outputs, handed):
        assert torch.allclose(got.double().cpu(), want, atol=2e-4, rtol=1e-4)


def test_borrowed_weights_are_shared_and_states_are_not():
    """Layers 4 and 5 run with the tensors of layers 1 and 2 -- through a chain and from a later layer too -- on caches and
    states of their own: the result differs from running the stack without them and equals the plain evaluation."""
    layers = [dict(DELTA, weights_of=2), LAT2, dict(DELTA, weights_of=3), DELTA, dict(LAT2, weights_of=1)]
    cfg = make_cfg(layers)
    W = O.random_weights(cfg, seed=6)
    assert not any(k.startswith(("l0.", "l2.", "l4.")) for k in W)
    toks = tokens(31, cfg["vocab"], 7)
    want = O.forward(cfg, W, toks)
    eng = make_engine(cfg, W)
    lw = eng.model().weights["layers"]
    assert lw[0] is lw[2] is lw[3] and lw[4] is lw[1]
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [5, 1, 2, 1]), want)


# ------------------------------------------------------------------------------------------------ cache, state, batches
def test_prefill_equals_token_by_token_decoding(stack):
    W, toks, want = stack
    eng = make_engine(STACK, W)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [1]), want)


@pytest.mark.parametrize("sizes", [[2], [3, 5], [7, 1, 1, 2], [16, 2, 9], [40, 1], [1, 2]])
def test_prompt_portions(stack, sizes):
    W, toks, want = stack
    eng = make_engine(STACK, W)
    close(feed(eng, 1, toks, sizes), want)


def test_unequal_requests_in_one_batch_equal_each_alone():
    W = O.random_weights(STACK, seed=9)
    reqs = {u: tokens(n, STACK["vocab"], 10 + u) for u, n in ((1, 19), (2, 3), (3, 31), (4, 8))}
    want = {u: O.forward(STACK, W, t) for u, t in reqs.items()}
    eng = make_engine(STACK, W)
    at = {u: 0 for u in reqs}
    got = {u: [] for u in reqs}
    plan = [{1: 5, 3: 2}, {1: 1, 2: 3, 3: 9, 4: 2}, {1: 13, 3: 1, 4: 1}, {3: 1, 4: 5}, {3: 18}]   # 2 is left out, 1 ends
    for step in plan:
        uids = list(step)
        toks = [torch.tensor(reqs[u][at[u]: at[u] + n]) for u, n in step.items()]
        out = eng.put(uids, toks, logit_positions=[list(range(n)) for n in step.values()]).double().cpu()
        k = 0
        for u, n in step.items():
            got[u].append(out[k: k + n])
            k, at[u] = k + n, at[u] + n
    for u in reqs:
        assert at[u] == len(reqs[u])
        close(torch.cat(got[u]), want[u])


def test_pages_and_state_slots_are_reused():
    """As many pages as the longest request and its neighbour need, two state slots: every later request gets pages and
    a slot that an earlier one filled, in another order, and must come out as if alone."""
    W = O.random_weights(STACK, seed=3)
    eng = make_engine(STACK, W, blocks=10, block_size=4, max_live=2)
    for i in range(4):
        toks = tokens(20 + 3 * i, STACK["vocab"], 20 + i)
        other = tokens(6, STACK["vocab"], 40 + i)
        eng.put([100 + i], [torch.tensor(other)])                 # a neighbour that holds the other slot and two pages
        got = feed(eng, i, toks, [7, 1, 2])
        close(got, O.forward(STACK, W, toks))
        eng.flush(i)
        eng.flush(100 + i)
        assert eng.free_blocks == 10


def test_far_keys_and_old_writes_decide_the_logits():
    """Attention with its score scale raised tenfold, so that single keys carry most of a query's weight wherever they
    lie among hundreds, and a delta rule whose channels barely decay, so that what the first tokens wrote is still read
    at the end: prompt rows, portions cut at page borders and beside them, and decode tokens follow the plain evaluation."""
    lat = dict(LAT, mixer=dict(LAT["mixer"], scale=3.0), mlp=None)
    lat2 = dict(LAT2, mixer=dict(LAT2["mixer"], scale=4.0), mlp=None)
    cfg = make_cfg([lat, dict(DELTA, mlp=None), lat2], vocab=31)
    W = O.random_weights(cfg, seed=21)
    W["l1.mix.A_log"] = torch.full_like(W["l1.mix.A_log"], -6.0)
    toks = tokens(300, cfg["vocab"], 22)
    want = O.forward(cfg, W, toks)
    eng = make_engine(cfg, W, block_size=8, blocks=128, max_tokens=320)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [245] + [1] * 55), want)
    close(feed(eng, 3, toks, [64, 37, 3, 2, 40, 4, 128, 7, 15]), want)
    # the far past matters: the same last tokens behind another beginning give other logits
    other = tokens(40, cfg["vocab"], 23) + toks[40:]
    assert (O.forward(cfg, W, other)[-1] - want[-1]).abs().max() > 1e-2


def test_long_decoding(stack):
    W, _, _ = stack
    toks = tokens(150, STACK["vocab"], 6)
    want = O.forward(STACK, W, toks)
    eng = make_engine(STACK, W)
    close(feed(eng, 1, toks, [9] + [1] * 200), want)


ODD = [
    # nothing a multiple of 8; one head; one expert chosen of one group; rotation of part of the rotated channels
    make_cfg([{"type": "latent_attention",
               "mixer": {"dim": 5, "heads": 1, "kv_rank": 7, "q_rank": 3, "rot": {"base": 77.0, "dims": 4}, "rot_dim": 6,
                         "scale": 1.7, "vdim": 3},
               "mlp": {"expert": {"ff": 7, "limit": 0.5}, "kind": "moe",
                       "router": {"experts": 3, "groups": {"count": 1, "keep": 1}, "identity": 0, "scale": 1.0, "top": 1}}},
              {"type": "channel_delta", "mixer": {"conv": 2, "dim": 5, "heads": 3, "kv_heads": 1, "vdim": 3},
               "mlp": {"ff": 9, "kind": "dense"}}], width=10, vocab=17, eps=1e-3),
    # long filter, one tap less than the first portions; as many identity experts as real ones; every group kept
    make_cfg([{"type": "channel_delta", "mixer": {"conv": 6, "dim": 33, "heads": 2, "kv_heads": 2, "vdim": 40},
               "mlp": {"expert": {"ff": 64, "limit": 3.0}, "kind": "moe",
                       "router": {"experts": 2, "groups": {"count": 2, "keep": 2}, "identity": 2, "scale": 0.7, "top": 4}}},
              {"type": "latent_attention_2",
               "mixer": {"dim": 16, "heads": 8, "kv_rank": 24,
                         "rot": {"base": 1e4, "dims": 4, "scaling": {"factor": 16.0, "fast": 2.0, "original": 8,
                                                                      "slow": 0.25}},
                         "rot_dim": 4, "scale": 0.2, "vdim": 4}, "mlp": None}], width=64, vocab=29),
    # a stack of one kind; a taps-1 filter; a single key channel group shared by all heads
    make_cfg([{"type": "channel_delta", "mixer": {"conv": 1, "dim": 4, "heads": 4, "kv_heads": 1, "vdim": 4},
               "mlp": None}] * 2 + [{"type": "channel_delta", "weights_of": 0,
                                     "mixer": {"conv": 1, "dim": 4, "heads": 4, "kv_heads": 1, "vdim": 4}, "mlp": None}],
             width=8, vocab=11),
    # no rotation at all; a latent wider than the heads; two layers of attention only
    make_cfg([{"type": "latent_attention",
               "mixer": {"dim": 4, "heads": 2, "kv_rank": 36, "q_rank": 40, "rot": {"base": 10.0, "dims": 0},
                         "rot_dim": 2, "scale": 0.5, "vdim": 6}, "mlp": {"ff": 5, "kind": "dense"}},
              dict(LAT2, mlp=MOE)], width=16, vocab=23),
]


@pytest.mark.parametrize("cfg", ODD, ids=["no_multiples_of_8_one_head_top_1", "long_filter_identity_experts_all_groups",
                                          "delta_only_one_tap_one_key_group", "no_rotation_wide_latent"])
def test_other_sizes(cfg):
    W = O.random_weights(cfg, seed=8, rank=3 if cfg["width"] == 10 else 8)
    toks = tokens(21, cfg["vocab"], 9)
    want = O.forward(cfg, W, toks)
    eng = make_engine(cfg, W, block_size=8)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [4, 1, 2]), want)


def test_configuration_is_read_into_the_layer_specs():
    from shuffle_exchange_b200.inference.v2.checkpoint.huggingface_engine import PlainModelConfig
    from shuffle_exchange_b200.inference.v2.model_implementations.pifazen import PifazenPolicy
    spec = PifazenPolicy(PlainModelConfig(STACK)).spec(PlainModelConfig(STACK))
    a, b, c, d, e, f = spec.layers
    assert (a.kind, a.n_heads, a.key_dim, a.value_dim, a.kv_rank, a.rot_dim, a.rot_dims, a.rot_base, a.attn_scale) == (
        "latent_attention", 4, 4, 8, 12, 8, 8, 200.0, 0.4)
    assert a.q_direct and a.gate_per_head and a.out_gate and a.rot_scaling == (4.0, 16.0, 4.0, 1.0) and not a.sink
    assert (a.ff_kind, a.ff_dim, a.ff_activation) == ("biased", 40, "power_norm")
    assert (b.kind, b.n_heads, b.n_heads_kv, b.key_dim, b.value_dim, b.conv_taps) == ("channel_delta", 4, 2, 8, 12, 3)
    assert (b.ff_kind, b.ff_dim, b.n_experts, b.top_k, b.moe_identity, b.moe_groups, b.moe_keep_groups, b.moe_scale,
            b.ff_limit, b.ff_activation, b.moe_correction) == ("moe", 16, 6, 3, 2, 4, 2, 1.5, 1.5, "clamped_swish", True)
    assert (c.q_rank, c.q_direct, c.gate_per_head, c.rot_scaling, c.window) == (12, False, False, None, 0)
    assert d.ff_dim == 0 and e.kind == "channel_delta" and f.kind == "latent_attention"
    assert (spec.block_form, spec.layer_scale, spec.norm_weight_offset, spec.residual_mult) == ("pre_scaled", True, 1.0, 1.0)
    assert len(spec.runs()) == 6


def test_bf16_serving_stays_near_the_exact_evaluation(stack):
    W, toks, want = stack
    eng = make_engine(STACK, W, dtype=torch.bfloat16)
    for uid, sizes in ((1, [len(toks)]), (2, [5, 1, 2])):
        d = feed(eng, uid, toks, sizes) - want
        err = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / want.std()
        # a token whose best experts score nearly alike may be routed otherwise in 16-bit: a few rows may differ
        assert err.median() < 0.03 and (err > 0.12).sum() <= 3, err


# ------------------------------------------------------------------------------------------------ generation
def _check_greedy(prompt, out, W, cfg):
    seq = list(prompt)
    for tok in out:
        logits = O.forward(cfg, W, seq)[-1]
        top2 = logits.topk(2).values
        if top2[0] - top2[1] > 1e-3:                           # a near tie may go either way in 32-bit
            assert tok == int(logits.argmax())
        seq.append(tok)


def test_greedy_generation_through_the_scheduler():
    W = O.random_weights(STACK, seed=12)
    prompts = [tokens(n, STACK["vocab"], 30 + n) for n in (5, 17, 2, 9, 12)]          # five requests, four may be live
    eng = make_engine(STACK, W, blocks=40, block_size=4, max_live=4, max_tokens=16)
    got = generate(eng, prompts, max_new_tokens=6, max_batch_tokens=16, max_prompt_portion=7)
    for p, out in zip(prompts, got):
        _check_greedy(p, out, W, STACK)
        assert len(out) == 6
    assert eng.free_blocks == 40 and eng._state_manager.n_tracked_sequences == 0


def write_checkpoint(folder, cfg, W):
    """``config.json`` + ``model.safetensors`` (bf16): 8-byte header length, JSON header, tensor bytes."""
    import json
    import struct
    with open(folder / "config.json", "w") as f:
        json.dump(cfg, f)
    meta, blobs, off = {}, [], 0
    for name, t in W.items():
        b = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        meta[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    header = json.dumps(meta).encode()
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + b"".join(blobs))


def test_command_line_generation_from_a_checkpoint_folder(tmp_path):
    """``bin/sxb_generate`` picks the model class by the configuration, loads the tensors by their checkpoint names and
    continues two prompts greedily."""
    import json
    import os
    import subprocess
    import sys
    W = O.random_weights(STACK, seed=14)
    write_checkpoint(tmp_path, STACK, W)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompts = [[5, 17, 3], [9, 9, 1, 2, 3, 4, 5, 6, 7]]
    cmd = [sys.executable, os.path.join(root, "bin", "sxb_generate"), "--model", str(tmp_path), "--max-new-tokens", "4",
           "--dtype", "float32"]
    for p in prompts:
        cmd += ["--prompt", ",".join(map(str, p))]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(x) for x in r.stdout.splitlines() if x.startswith("{")]
    assert [x["prompt"] for x in lines] == prompts
    for p, x in zip(prompts, lines):
        _check_greedy(p, x["generated"], W, STACK)
        assert len(x["generated"]) == 4


def test_replaying_a_schedule_of_steps_from_a_checkpoint_folder(tmp_path):
    """``bin/trace_run``: five requests through a pool of four 64-token pages and four state slots -- portions beside single tokens, a
    request left out of a step, requests that end and whose pages and slot the next one takes -- write the logits of the
    wanted positions per step; every one must equal the plain evaluation of its request alone."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    W = O.random_weights(STACK, seed=15)
    model = tmp_path / "model"
    model.mkdir()
    write_checkpoint(model, STACK, W)
    reqs = {name: tokens(n, STACK["vocab"], 50 + n) for name, n in (("a", 40), ("b", 9), ("c", 23), ("d", 1), ("e", 30))}
    plan = [({"a": 17, "b": 2}, []), ({"a": 3, "b": 7, "c": 5, "d": 1}, ["b", "d"]), ({"a": 1, "c": 2, "e": 11}, []),
            ({"a": 19, "e": 1}, ["a"]), ({"c": 16, "e": 18}, ["c", "e"])]
    at = {k: 0 for k in reqs}
    steps, wanted = [], []
    for i, (portion, end) in enumerate(plan):
        entries = []
        for name, n in portion.items():
            want = sorted({0, n - 1, n // 2})
            entries.append({"id": name, "tokens": reqs[name][at[name]: at[name] + n], "want": want})
            wanted += [(i, name, at[name] + w) for w in want]
            at[name] += n
        steps.append(json.dumps({"step": i, "entries": entries, "end": end}))
    assert at == {k: len(v) for k, v in reqs.items()}
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    cmd = [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model), "--dtype", "float32", "--out",
           str(out), "--max-tokens", "256"] + ([] if torch.cuda.is_available() else ["--device", "cpu"])
    r = subprocess.run(cmd, input="\n".join(steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [x for x in r.stdout.splitlines() if x.startswith("done")] == [f"done {i}" for i in range(len(plan))]
    full = {name: O.forward(STACK, W, t) for name, t in reqs.items()}
    got = {i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, STACK["vocab"])).double()
           for i in range(len(plan))}
    row = {i: 0 for i in got}
    for i, name, p in wanted:
        close(got[i][row[i]: row[i] + 1], full[name][p: p + 1])
        row[i] += 1
    assert all(row[i] == got[i].shape[0] for i in got)
