"""The Pifazen cases of ``test_pifazen.py`` on the CUDA kernels (``csrc/seq_mixers.cu``, ``csrc/moe_ragged.cu``): the same
functions, collected here under the ``gpu`` marker; the ops take their kernel branch because their tensors live on the
device."""
import pytest
import torch

from test_pifazen import *  # noqa: F401,F403  (collects every test of that module again)
from test_pifazen import DELTA, LAT, LAT2, MOE, O, close, feed, make_cfg, make_engine, tokens
from shuffle_exchange_b200.native import lib as _lib

pytestmark = pytest.mark.gpu


def test_the_kernels_ran():
    from shuffle_exchange_b200.inference.v2.kernels import mixer_ops as M
    before = _lib.launch_count
    x = torch.ones(3, 16, device="cuda")
    M.sigmoid_gate_rows_(x, torch.zeros(3, 16, device="cuda"), 1)
    assert _lib.launch_count == before + 1
    assert torch.allclose(x, torch.full_like(x, 0.5))


def test_prompts_on_the_tiled_kernel_and_experts_on_the_grouped_gemm_path():
    """Widths that are multiples of 64 in bf16 take the grouped tensor-core path of the experts, where the identity
    experts' row groups are copied between the two products; prompts of more than 16 tokens take the tiled attention
    kernel on the latent rows."""
    moe = dict(MOE, expert={"ff": 64, "limit": 1.5})
    layers = [dict(LAT, mixer=dict(LAT["mixer"], dim=16, vdim=32, kv_rank=40, q_rank=24), mlp=moe),
              dict(DELTA, mixer=dict(DELTA["mixer"], dim=32, vdim=32), mlp=moe),
              dict(LAT2, mixer=dict(LAT2["mixer"], dim=16, vdim=16, kv_rank=56),
                   mlp=dict(moe, expert={"ff": 128, "limit": 4.0},
                            router={"experts": 3, "top": 2, "identity": 1, "groups": {"count": 2, "keep": 1}, "scale": 2.0}))]
    cfg = make_cfg(layers, width=64)
    W = O.random_weights(cfg, seed=31, rank=8)
    toks = tokens(150, cfg["vocab"], 32)
    want = O.forward(cfg, W, toks)
    eng = make_engine(cfg, W, dtype=torch.bfloat16, max_tokens=256, blocks=128)
    for sizes in ([len(toks)], [70, 1, 33, 1, 1]):
        d = feed(eng, len(sizes), toks, sizes) - want
        err = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / want.std()
        assert err.median() < 0.03 and (err > 0.12).sum() <= 8, err
    eng32 = make_engine(cfg, W, dtype=torch.float32, max_tokens=256, blocks=128)
    close(feed(eng32, 1, toks, [len(toks)]), want)
    close(feed(eng32, 2, toks, [70, 1, 33, 1, 1]), want)


def test_identity_rows_are_copied_between_the_grouped_products():
    """Every token sends one row to an identity expert (its correction is far above the others): with two experts chosen
    the result is ``w_id * x + w_e * expert(x)``, on the grouped path in bf16."""
    from test_pifazen import _experts  # noqa: F401
    from shuffle_exchange_b200.inference.v2.inference_utils import ActivationType, DtypeEnum
    from shuffle_exchange_b200.inference.v2.modules import heuristics
    from shuffle_exchange_b200.inference.v2.modules.configs import DSMoEConfig
    g = torch.Generator().manual_seed(5)
    T, Wd, Fe, E, n_id = 200, 64, 64, 3, 2
    h = (torch.randn(T, Wd, generator=g)).to(torch.bfloat16)
    P = {"router": torch.randn(E + n_id, Wd, generator=g), "correction": torch.tensor([0.0, 0.0, 0.0, 0.0, 9.0])}
    for e in range(E):
        P[f"e{e}.gate"] = (torch.randn(Fe, Wd, generator=g) / 4).to(torch.bfloat16)
        P[f"e{e}.up"] = (torch.randn(Fe, Wd, generator=g) / 4).to(torch.bfloat16)
        P[f"e{e}.down"] = (torch.randn(Wd, Fe, generator=g) / 4).to(torch.bfloat16)
    mlp = {"router": {"experts": E, "identity": n_id, "top": 2, "groups": {"count": 1, "keep": 1}, "scale": 1.0},
           "expert": {"ff": Fe, "limit": 2.0}}
    mod = heuristics.instantiate_moe(DSMoEConfig(
        max_tokens=256, model_dim=Wd, intermediate_features=Fe, n_experts=E, top_k=2, input_dtype=DtypeEnum.bf16,
        output_dtype=DtypeEnum.bf16, activation=ActivationType.CLAMPED_SWIGLU, router_dtype=DtypeEnum.fp32,
        score_correction=True, identity_experts=n_id, activation_limit=2.0), None)
    w1 = torch.stack([torch.cat([P[f"e{e}.gate"], P[f"e{e}.up"]]) for e in range(E)]).cuda()
    w2 = torch.stack([P[f"e{e}.down"] for e in range(E)]).cuda()
    before = _lib.launch_count
    got = mod(h.cuda(), P["router"].cuda(), w1, w2, correction=P["correction"].cuda()).double().cpu()
    assert _lib.launch_count > before
    want = O.expert_ff(h.double(), {k: v.double() for k, v in P.items()}, mlp)
    assert (got - want).abs().max() < 0.05 * want.abs().max(), float((got - want).abs().max())


def test_a_latent_wider_than_the_kernels_value_tile():
    layer = dict(LAT, mixer=dict(LAT["mixer"], kv_rank=264, rot_dim=8, rot={"base": 1000.0, "dims": 8}), mlp=None)
    cfg = make_cfg([layer, dict(LAT2, mixer=dict(LAT2["mixer"], kv_rank=300), mlp=None)], width=32)
    W = O.random_weights(cfg, seed=41)
    toks = tokens(40, cfg["vocab"], 42)
    want = O.forward(cfg, W, toks)
    eng = make_engine(cfg, W, max_tokens=64)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [19, 1, 2]), want)


def test_other_sizes_in_bf16():
    """Widths and head sizes that are not multiples of 8 take the scalar forms of the kernels and the library products;
    16-bit serving must still follow the exact evaluation."""
    from test_pifazen import ODD
    for cfg in ODD:
        W = O.random_weights(cfg, seed=8, rank=3 if cfg["width"] == 10 else 8)
        toks = tokens(40, cfg["vocab"], 9)
        want = O.forward(cfg, W, toks)
        eng = make_engine(cfg, W, dtype=torch.bfloat16, block_size=8)
        for uid, sizes in ((1, [len(toks)]), (2, [19, 1, 2])):
            d = feed(eng, uid, toks, sizes) - want
            err = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / want.std()
            assert err.median() < 0.04 and (err > 0.15).sum() <= 4, err
