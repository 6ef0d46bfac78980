"""Helpers of the Motolix tests: small made-up configurations, random weights, the oracle's logits and engines built from
them.  The step driver (Feeder) and the error measures are those of the other layer-list tests."""
import copy

import numpy as np

from distributed_inference_server_b200 import Engine, WorkerConfig, models
from tests import motolix_oracle as MO
from tests._stack_util import Feeder, bf16_close, rel_err, row_errs  # noqa: F401  (re-exported)


def attention(heads=4, kv_heads=2, dim=8, rot_dims=4, base=10000.0, scale=None, scaling=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "rot": rot,
                                           "scale": dim ** -0.5 if scale is None else scale}}


def parallel(heads=4, kv_heads=2, dim=8, vdim=12, rot_dims=6, base=5000.0, scale=None, left_scale=0.7, right_scale=1.1,
             r_heads=3, r_dim=8, r_vdim=12, tau=4.0, rank=5):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot_dims},
            "scale": dim ** -0.5 if scale is None else scale}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "tau": tau, "rank": rank}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff=24):
    return {"kind": "dense", "ff": ff}


def config(layers, vocab=50, width=32, eps=1e-5, loop=None, embed_scale=3.0, logit_scale=0.5):
    """layers: list of (mixer dict, mlp dict or None); loop: (start, stop, times) or None."""
    cfg = {"architecture": "Motolix", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": embed_scale}, "logit_scale": logit_scale, "layers": [dict(copy.deepcopy(m), mlp=copy.deepcopy(f)) for m, f in layers]}
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


def weights(cfg, seed=0, gain=1.0):
    """Random float32 tensors by name, every value representable in bfloat16 (both compute types then see one model)."""
    spec = models.motolix_spec(cfg)
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in spec.tensor_shapes().items():
        leaf = name.rsplit(".", 1)[-1]
        if name.endswith("a2.b"):
            a = rng.normal(1.5, 1.5, shape)
        elif leaf == "b" and ".norm" in name:
            a = rng.normal(0, 0.2, shape)
        elif leaf == "b":
            a = rng.normal(0, 0.5, shape)
        elif leaf in ("norm1", "norm1b", "norm2", "norm2b", "norm", "temp"):
            a = rng.uniform(0.5, 1.5, shape)
        elif leaf == "pb":
            a = rng.normal(-1.5, 1.0, shape)
        elif name == "loop.step":
            a = rng.normal(0, 0.3, shape)
        elif name == "embed":
            a = rng.normal(0, 1.0, shape)
        else:
            a = rng.normal(0, gain / np.sqrt(shape[-1]), shape)
        out[name] = models.bf16_round(np.asarray(a, np.float32))
    return out


def oracle_logits(cfg, W, tokens, layers_out=None):
    return MO.forward(cfg, W, tokens, layers_out)


def engine(cfg, W, dtype="float32", max_batch=4, pool_tokens=512, page_size=8, max_step_tokens=0, rows=0):
    spec = models.motolix_spec(cfg)
    cap = max_step_tokens or pool_tokens
    e = Engine(WorkerConfig(None, max_batch=max_batch, max_step_tokens=cap, page_size=page_size,
                            kv_pages=(pool_tokens + page_size - 1) // page_size, stack=spec, context_size=pool_tokens + page_size,
                            compute_dtype=dtype, max_logit_rows=(rows or cap) + max_batch))
    for name, a in W.items():
        e.load_named(name, np.asarray(a, np.float32))
    e.finalize()
    return e


def run_whole(cfg, W, tokens, dtype="float32", **kw):
    e = engine(cfg, W, dtype, **kw)
    f = Feeder(e)
    f.step([("a", tokens, len(tokens))])
    out = f.end("a")
    e.close()
    return out


def run_portions(cfg, W, tokens, sizes, dtype="float32", **kw):
    """The sequence in portions of the given sizes (the rest one token at a time)."""
    e = engine(cfg, W, dtype, **kw)
    f = Feeder(e)
    fed = 0
    for n in sizes:
        n = min(n, len(tokens) - fed)
        if n <= 0:
            break
        f.step([("a", tokens, n)])
        fed += n
    while fed < len(tokens):
        f.step([("a", tokens, 1)])
        fed += 1
    out = f.end("a")
    e.close()
    return out
