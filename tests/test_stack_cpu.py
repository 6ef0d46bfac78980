"""CPU-side checks of the layer-list family: the configuration reader, the tensor name table, the safetensors reader, the
registry, and the layout of the C structs that describe a layer list."""
import ctypes as C
import json
import os
import struct
import subprocess

import numpy as np
import pytest
import torch

from distributed_inference_server_b200 import binding as B
from distributed_inference_server_b200 import models
from tests import _stack_util as U
from tests import kidolorn_oracle as KO

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def write_safetensors(path, tensors):
    """name -> float32 array; stored as bfloat16 bit patterns (values must be representable)."""
    header, blobs, at = {}, [], 0
    for name, a in tensors.items():
        shape = list(np.shape(a))
        a = np.ascontiguousarray(a, np.float32).reshape(-1)
        bits = (a.view(np.uint32) >> 16).astype(np.uint16)
        assert np.array_equal((bits.astype(np.uint32) << 16).view(np.float32), a), name
        raw = bits.tobytes()
        header[name] = {"dtype": "BF16", "shape": shape, "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


CFG = U.config([(U.latent(), U.moe(ff=6, experts=5, top=3)), (U.mingru(28), U.moe()),
                (U.lightning(heads=3, dim=4, vdim=8), U.dense(ff=20, limit=0.75)), (U.latent(kv_from=0, vdim=6), None)],
               vocab=77, width=24, taps=2, eps=3e-4)


def test_config_reader_takes_every_size_and_constant_from_the_file():
    s = models.kidolorn_spec(CFG)
    assert (s.vocab, s.width, s.canon_taps, len(s.layers)) == (77, 24, 2, 4) and abs(s.norm_eps - 3e-4) < 1e-12
    b, d, a, c = s.layers
    assert (a.mixer, a.heads, a.dim, a.vdim, a.mlp, a.ff, a.limit) == ("lightning", 3, 4, 8, "dense", 20, 0.75) and len(a.decay) == 3
    assert (b.mixer, b.kv_rank, b.rot_dim, b.rot_dims, b.kv_from, b.mlp, b.experts, b.top, b.ff) == ("latent_attention", 16, 4, 4, -1, "moe", 5, 3, 6)
    assert (c.kv_from, c.vdim, c.mlp) == (0, 6, "none")
    assert (d.mixer, d.width, d.limit) == ("mingru", 28, 1.25)
    assert models.kidolorn_spec(U.config([(U.mingru(), None)], taps=0)).canon_taps == 0


def test_tensor_table_is_what_the_plain_implementation_reads():
    """The oracle runs on exactly the tensors the table names (a missing one raises KeyError, shapes must multiply)."""
    W = U.weights(CFG, seed=1)
    names = set(models.kidolorn_spec(CFG).tensor_shapes())
    assert "l3.mix.dkv" not in names and "l0.mix.dkv" in names and "l3.norm2" not in names and "l1.mlp.e3.down" in names
    out = KO.forward(CFG, {k: torch.from_numpy(v.copy()) for k, v in W.items()}, [1, 2, 3, 4, 5])
    assert out.shape == (5, 77) and bool(torch.isfinite(out).all())


def test_safetensors_reader_round_trip(tmp_path):
    W = U.weights(CFG, seed=2)
    write_safetensors(tmp_path / "model.safetensors", W)
    got = {n: (a, code, shape) for n, a, code, shape in models.read_safetensors(str(tmp_path / "model.safetensors"))}
    assert set(got) == set(W)
    for n, (a, code, shape) in got.items():
        assert code == B.BF16 and shape == W[n].shape
        assert np.array_equal((a.astype(np.uint32) << 16).view(np.float32).reshape(shape), W[n])


def test_registry_picks_the_family_by_config(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    fam, spec = models.read_config(str(tmp_path))
    assert fam == "stack" and spec.name == "Kidolorn"
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["LlamaForCausalLM"], "vocab_size": 100, "hidden_size": 64,
                                                      "num_hidden_layers": 2, "num_attention_heads": 4, "intermediate_size": 128}))
    fam, shape = models.read_config(str(tmp_path))
    assert fam == "llama" and (shape.vocab, shape.head_dim, shape.n_kv_heads) == (100, 16, 4)
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nothing"}))
    with pytest.raises(ValueError):
        models.read_config(str(tmp_path))
    with pytest.raises(ValueError):
        models.kidolorn_spec(U.config([({"type": "conv", "mixer": {}}, None)]))


def test_bf16_round_is_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.1415927, 0.0], np.float32)  # 1 + 2^-8 is a tie: rounds to even (1.0)
    assert np.array_equal(models.bf16_round(x), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


def test_stack_structs_match_the_header(tmp_path):
    probe = tmp_path / "probe.c"
    probe.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "dis_engine.h"\nint main(){printf("%zu %zu %zu %zu %zu %zu\\n",'
                     'sizeof(dis_layer_config),sizeof(dis_stack_config),offsetof(dis_layer_config,decay),offsetof(dis_layer_config,limit),'
                     'offsetof(dis_stack_config,norm_eps),offsetof(dis_stack_config,layers));return 0;}\n')
    exe = tmp_path / "probe"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(probe), "-o", str(exe)], check=True)
    sizes = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    assert sizes == [C.sizeof(B.LayerConfig), C.sizeof(B.StackConfig), B.LayerConfig.decay.offset, B.LayerConfig.limit.offset,
                     B.StackConfig.norm_eps.offset, B.StackConfig.layers.offset]


def test_trace_runner_is_an_executable_of_the_checkout():
    p = os.path.join(ROOT, "bin", "trace_run")
    assert os.path.isfile(p) and os.access(p, os.X_OK)
