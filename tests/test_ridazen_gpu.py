"""The Ridazen cases of ``test_ridazen.py`` on the CUDA kernels (``csrc/seq_mixers.cu``, ``csrc/moe_ragged.cu``): the same
functions, collected here under the ``gpu`` marker; the ops take their kernel branch because their tensors live on the
device."""
import pytest
import torch

from test_ridazen import *  # noqa: F401,F403  (collects every test of that module again)
from test_ridazen import ATT, MOE, O, feed, make_cfg, make_engine, tokens
from shuffle_exchange_b200.native import lib as _lib

pytestmark = pytest.mark.gpu


def test_the_kernels_ran():
    from shuffle_exchange_b200.inference.v2.kernels import mixer_ops as M
    before = _lib.launch_count
    z = torch.full((3, 10), 40.0, device="cuda")
    M.scale_softcap_(z, 0.5, 4.0)
    assert _lib.launch_count == before + 1
    assert torch.allclose(z, torch.full_like(z, 4.0), atol=1e-3)


def test_prompts_on_the_tiled_kernel_and_experts_on_the_grouped_gemm_path():
    """Widths that are multiples of 64 in bf16 take the grouped tensor-core path of the experts; prompts of more than 16
    tokens take the tiled attention kernel, where the distance bias and the gate are applied per tile."""
    layers = [dict(ATT, mixer=dict(ATT["mixer"], dim=16, vdim=32, bias_max=60),
                   mlp=dict(MOE, expert={"ff": 64}, shared={"ff": 32})),
              dict(ATT, mlp=dict(MOE, expert={"ff": 128}, router={"experts": 3, "top": 1}, shared=None))]
    cfg = make_cfg(layers, width=64)
    W = O.random_weights(cfg, seed=31)
    toks = tokens(150, cfg["vocab"], 32)
    want = O.forward(cfg, W, toks)
    eng = make_engine(cfg, W, dtype=torch.bfloat16, max_tokens=256, blocks=128)
    for sizes in ([len(toks)], [70, 1, 33, 1, 1]):
        d = feed(eng, len(sizes), toks, sizes) - want
        err = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / want.std()
        assert err.median() < 0.02 and (err > 0.08).sum() <= 7, err
    eng32 = make_engine(cfg, W, dtype=torch.float32, max_tokens=256)
    d = feed(eng32, 1, toks, [len(toks)]) - want
    assert (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt().max() / want.std() < 2e-4


def test_other_sizes_in_bf16():
    """Widths and head sizes that are not multiples of 8 take the scalar forms of the kernels and the library products;
    16-bit serving must still follow the exact evaluation."""
    from test_ridazen import ODD
    for cfg in ODD:
        W = O.random_weights(cfg, seed=8, rel_rows=2 + 2 * len(cfg["layers"]))
        toks = tokens(40, cfg["vocab"], 9)
        want = O.forward(cfg, W, toks)
        eng = make_engine(cfg, W, dtype=torch.bfloat16, block_size=8)
        for uid, sizes in ((1, [len(toks)]), (2, [19, 1, 2])):
            d = feed(eng, uid, toks, sizes) - want
            err = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / want.std()
            assert err.median() < 0.03 and (err > 0.12).sum() <= 4, err
