"""Motolix without a GPU: the configuration reader, the table of tensor names and shapes, the order of layer runs, and the
oracle's own sensitivity to every constant the GPU tests rely on."""
import numpy as np

from distributed_inference_server_b200 import binding as B
from distributed_inference_server_b200 import models
from tests import _motolix_util as U


def toks(n, vocab=50, seed=0):
    return [int(x) for x in np.random.default_rng(seed).integers(0, vocab, n)]


def test_registry_reads_the_configuration():
    cfg = U.config([(U.parallel(), U.dense()), (U.attention(scaling=(8.0, 1.0, 4.0, 16)), None)], loop=(0, 2, 3), width=40, vocab=77)
    assert models.architecture_of(cfg) == "Motolix"
    family, reader = models.ARCHITECTURES["Motolix"]
    spec = reader(cfg)
    assert family == "stack" and spec.norm_kind == "layer" and spec.loop == (0, 2, 3)
    assert spec.embed_scale == 3.0 and spec.logit_scale == 0.5 and spec.layer_runs() == [0, 1, 0, 1, 0, 1]
    p, a = spec.layers
    assert p.mixer == "parallel" and p.attn_flags == B.ATTN_QK_NORM | B.ATTN_ROT_V and (p.heads, p.kv_heads, p.dim, p.vdim) == (4, 2, 8, 12)
    assert (p.gla_heads, p.gla_dim, p.gla_vdim, p.gla_rank, p.gla_tau) == (3, 8, 12, 5, 4.0) and (p.mix_scale, p.gla_scale) == (0.7, 1.1)
    assert p.mlp == "dense" and p.mlp_act == "gelu_tanh" and a.mlp == "none"
    assert a.attn_flags == B.ATTN_SIGMOID | B.ATTN_V_IS_K | B.ATTN_BIAS and (a.rot_factor, a.rot_low, a.rot_high, a.rot_original) == (8.0, 1.0, 4.0, 16)
    sc, _keep = spec.c(256, 8, False)
    assert sc.loop_times == 3 and sc.norm_kind == B.NORM_LAYER and sc.layers[0].gla_rank == 5 and sc.layers[1].kv_heads == 2


def test_tensor_table():
    cfg = U.config([(U.parallel(), U.dense(ff=20)), (U.attention(), None)], loop=(1, 2, 2), width=40, vocab=77)
    shapes = models.motolix_spec(cfg).tensor_shapes()
    assert shapes["loop.in"] == (40, 80) and shapes["loop.step"] == (2, 40) and shapes["final.norm.b"] == (40,)
    assert shapes["l0.mix.left.q"] == (32, 40) and shapes["l0.mix.left.k"] == (16, 40) and shapes["l0.mix.left.v"] == (24, 40)
    assert shapes["l0.mix.left.q.norm"] == (32,) and shapes["l0.mix.left.o"] == (40, 48)
    assert shapes["l0.mix.right.a1"] == (5, 40) and shapes["l0.mix.right.a2"] == (24, 5) and shapes["l0.mix.right.norm"] == (12,)
    assert shapes["l0.mlp.down"] == (40, 20) and "l0.mlp.gate.b" not in shapes and "l1.norm2" not in shapes
    assert shapes["l1.mix.q.b"] == (32,) and shapes["l1.mix.temp"] == (4,) and "l1.mix.v" not in shapes
    # the rank of the decay projection may come from the model file instead of the configuration
    del cfg["layers"][0]["mixer"]["right"]["rank"]
    assert models.motolix_spec(cfg, {"l0.mix.right.a1": (7, 40)}).layers[0].gla_rank == 7


def test_the_oracle_reacts_to_every_constant():
    """The oracle itself reacts to every constant the tests above rely on (a constant that the engine and the oracle both
    ignored would pass unnoticed)."""
    t = toks(30, seed=2)
    base = U.config([(U.parallel(), U.dense()), (U.attention(scaling=(8.0, 1.0, 4.0, 16)), None)], loop=(0, 2, 2))
    W = U.weights(base, seed=4)
    ref = U.oracle_logits(base, W, t)
    for change in ("left_scale", "right_scale", "tau", "scaling", "loop", "logit_scale", "embed"):
        cfg = U.config([(U.parallel(), U.dense()), (U.attention(scaling=(8.0, 1.0, 4.0, 16)), None)], loop=(0, 2, 2))
        if change in ("left_scale", "right_scale"):
            cfg["layers"][0]["mixer"][change] *= 1.5
        elif change == "tau":
            cfg["layers"][0]["mixer"]["right"]["tau"] = 1.0
        elif change == "scaling":
            del cfg["layers"][1]["mixer"]["rot"]["scaling"]
        elif change == "loop":
            cfg["loop"]["times"] = 1
        elif change == "logit_scale":
            cfg["logit_scale"] = 1.0
        else:
            cfg["embedding"]["scale"] = 1.0
        W2 = {k: v for k, v in W.items() if k != "loop.step"}
        W2["loop.step"] = W["loop.step"][:cfg["loop"]["times"]]
        assert U.rel_err(U.oracle_logits(cfg, W2, t), ref) > 1e-3, change
