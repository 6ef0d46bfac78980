"""Helpers of the layer-list decoder tests: small made-up configurations, random weights, the oracle's logits, and a driver
that pushes token portions through the engine's step call and collects the logits of every position."""
import numpy as np
import torch

from distributed_inference_server_b200 import Engine, InferenceParams, WorkerConfig, models
from tests import kidolorn_oracle as KO


def lightning(heads=2, dim=8, vdim=16, decay=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim,
                                          "decay": decay or [0.5 + 0.49 * (h + 1) / heads for h in range(heads)]}}


def mingru(width=24):
    return {"type": "mingru", "mixer": {"width": width}}


def latent(heads=2, dim=8, rot_dim=4, vdim=12, kv_rank=16, kv_from=None, rot_dims=None, base=10000.0, scale=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
          "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
          "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mx}


def dense(ff=24, limit=2.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff=12, experts=4, top=2, limit=1.25):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def config(layers, vocab=50, width=32, taps=2, eps=1e-6):
    """layers: list of (mixer dict, mlp dict or None)."""
    cfg = {"architecture": "Kidolorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [dict(m, mlp=f) for m, f in layers]}
    if taps:
        cfg["canon"] = {"taps": taps}
    return cfg


def weights(cfg, seed=0, gain=1.0):
    """Random float32 tensors by name, every value representable in bfloat16 (both compute types then see one model)."""
    spec = models.kidolorn_spec(cfg)
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in spec.tensor_shapes().items():
        leaf = name.rsplit(".", 1)[-1]
        if shape == ():
            a = np.asarray(rng.uniform(0.6, 1.4), np.float32)
        elif leaf in ("canon1", "canon2"):
            a = rng.normal(0, 0.4, shape)
        elif leaf == "norm":
            a = rng.uniform(0.5, 1.5, shape)
        elif leaf in ("sink", "b"):
            a = rng.normal(0, 0.5, shape)
        elif name == "embed":
            a = rng.normal(0, 1.0, shape)
        else:
            a = rng.normal(0, gain / np.sqrt(shape[-1]), shape)
        out[name] = models.bf16_round(np.asarray(a, np.float32))
    return out


def oracle_logits(cfg, W, tokens, layers_out=None):
    tens = {k: torch.from_numpy(np.asarray(v, np.float32).copy()) for k, v in W.items()}
    return KO.forward(cfg, tens, tokens, torch.float64, layers_out).numpy()


def engine(cfg, W, dtype="float32", max_batch=4, pool_tokens=512, page_size=8, max_step_tokens=0, rows=0):
    spec = models.kidolorn_spec(cfg)
    cap = max_step_tokens or pool_tokens
    e = Engine(WorkerConfig(None, max_batch=max_batch, max_step_tokens=cap, page_size=page_size,
                            kv_pages=(pool_tokens + page_size - 1) // page_size, stack=spec, context_size=pool_tokens + page_size,
                            compute_dtype=dtype, max_logit_rows=(rows or cap) + max_batch))
    for name, a in W.items():
        e.load_named(name, np.asarray(a, np.float32))
    e.finalize()
    return e


class Feeder:
    """Feeds portions of given token sequences through Engine.step and keeps the logits of every position."""

    def __init__(self, eng):
        self.eng, self.slot, self.fed, self.out = eng, {}, {}, {}
        self.params = InferenceParams(max_tokens=1 << 30, temperature=0.0)

    def step(self, portions):
        """portions: list of (key, tokens of the sequence `key`, n) -- the next n tokens of each listed sequence, one pass."""
        listed = []
        for key, toks, n in portions:
            lo = self.fed.get(key, 0)
            part = [int(t) for t in toks[lo:lo + n]]
            assert len(part) == n
            if key not in self.slot:
                self.slot[key] = self.eng.seq_add(part, self.params)
                self.eng.seq_probe(self.slot[key], list(range(n)))
            else:
                self.eng.seq_extend(self.slot[key], part, list(range(n)))
            self.fed[key] = lo + n
            listed.append((key, n))
        _, _, prod = self.eng.step([self.slot[k] for k, _ in listed])
        assert all(prod), "the pass did not reach the end of every portion"
        rows = self.eng.last_logit_rows()
        assert rows == sum(n + 1 for _, n in listed)
        lg = self.eng.last_logits(rows)
        at = 0
        for key, n in listed:
            self.out.setdefault(key, []).extend(lg[at:at + n])
            assert np.allclose(lg[at + n - 1], lg[at + n], rtol=1e-5, atol=1e-6)  # the sampled row repeats the last position
            at += n + 1

    def end(self, key):
        self.eng.seq_remove(self.slot.pop(key))
        self.fed.pop(key)
        return np.stack(self.out.pop(key))

    def logits(self, key):
        return np.stack(self.out[key])


def row_errs(got, want):
    """Per row: root mean square of the difference (mean removed) over the root mean square of the wanted row."""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean(-1) + 1e-30)


def rel_err(got, want):
    return float(row_errs(got, want).max())


def bf16_close(got, want, tol=4e-2):
    """bfloat16 inputs can turn a close call of a router or a clamp the other way at single positions of these tiny random
    models, so the bulk of the rows must be close and no row may be wild."""
    e = row_errs(got, want)
    return float(np.quantile(e, 0.8)) < tol and float(e.max()) < 1.0


def run_whole(cfg, W, tokens, dtype="float32", **kw):
    e = engine(cfg, W, dtype, **kw)
    f = Feeder(e)
    f.step([("a", tokens, len(tokens))])
    out = f.end("a")
    e.close()
    return out
