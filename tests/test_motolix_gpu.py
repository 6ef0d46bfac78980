"""Motolix on the GPU against the float64 oracle (tests/motolix_oracle.py): small made-up configurations with random weights.
Covered: each mechanism alone, the residual stream layer by layer, prefill against token-by-token decoding, portions down to
two tokens, unequal batches, reuse of pages and slots, far keys / page borders / tile, slice and segment edges, the first
tokens, long decoding, other sizes, and greedy generation through the scheduler."""
import numpy as np
import pytest

from distributed_inference_server_b200 import ContinuousBatcher, InferenceParams, models
from tests import _motolix_util as U

pytestmark = pytest.mark.gpu
F32_TOL = 2e-5


def toks(n, vocab=50, seed=0):
    return [int(x) for x in np.random.default_rng(seed).integers(0, vocab, n)]


# the two halves of a parallel layer are isolated by giving the other half weight zero
MECHANISMS = {
    "sigmoid_attention": dict(layers=[(U.attention(), None)]),
    "sigmoid_attention_one_kv_head_full_rotary": dict(layers=[(U.attention(heads=3, kv_heads=1, dim=6, rot_dims=6), None)]),
    "sigmoid_attention_as_many_kv_heads_no_rotary": dict(layers=[(U.attention(heads=2, kv_heads=2, dim=10, rot_dims=0), None)]),
    "rotary_scaling_all_three_bands": dict(layers=[(U.attention(dim=16, rot_dims=16, base=10000.0, scaling=(8.0, 1.0, 4.0, 64)), None)]),
    "softmax_attention_rotated_values": dict(layers=[(U.parallel(right_scale=0.0), None)]),
    "softmax_attention_partial_rotary_one_group": dict(layers=[(U.parallel(heads=6, kv_heads=1, dim=12, vdim=6, rot_dims=4, right_scale=0.0), None)]),
    "gated_linear_attention": dict(layers=[(U.parallel(left_scale=0.0), None)]),
    "gated_linear_attention_fast_decay": dict(layers=[(U.parallel(left_scale=0.0, tau=0.5, r_heads=1, r_dim=20, r_vdim=4, rank=1), None)]),
    "parallel": dict(layers=[(U.parallel(), None)]),
    "feed_forward": dict(layers=[(U.attention(), U.dense())]),
    "loop_from_the_first_layer": dict(layers=[(U.attention(), U.dense()), (U.parallel(), None)], loop=(0, 1, 3)),
    "loop_to_the_last_layer_once": dict(layers=[(U.parallel(), None), (U.attention(), U.dense())], loop=(1, 2, 1)),
    "loop_over_all": dict(layers=[(U.parallel(), U.dense()), (U.attention(), None)], loop=(0, 2, 2)),
}


@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_alone(name):
    cfg = U.config(**MECHANISMS[name])
    W = U.weights(cfg, seed=3)
    t = toks(70, seed=1)
    want = U.oracle_logits(cfg, W, t)
    got = U.run_whole(cfg, W, t)
    assert U.rel_err(got, want) < F32_TOL
    got16 = U.run_whole(cfg, W, t, dtype="bfloat16")
    assert U.bf16_close(got16, want)


STACK = [(U.parallel(), U.dense()), (U.attention(scaling=(4.0, 1.0, 4.0, 32)), U.dense(ff=16)), (U.parallel(heads=2, kv_heads=2, r_heads=2), None),
         (U.attention(heads=2, kv_heads=1, dim=12, rot_dims=8), U.dense())]


def test_residual_stream_after_every_layer_matches():
    """Models cut after each layer (with the loop cut to what is left of it) reproduce the oracle layer by layer."""
    t = toks(40, seed=2)
    for n in range(1, len(STACK) + 1):
        cfg = U.config(STACK[:n], loop=(1, min(n, 3), 2) if n > 1 else None)
        W = U.weights(cfg, seed=5)
        assert U.rel_err(U.run_whole(cfg, W, t), U.oracle_logits(cfg, W, t)) < F32_TOL, n


FULL = dict(layers=STACK, loop=(1, 3, 2))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_against_token_by_token_decoding(dtype):
    cfg = U.config(**FULL)
    W = U.weights(cfg, seed=7)
    t = toks(48, seed=3)
    want = U.oracle_logits(cfg, W, t)
    whole = U.run_whole(cfg, W, t, dtype)
    single = U.run_portions(cfg, W, t, [], dtype)
    if dtype == "float32":
        assert U.rel_err(whole, want) < F32_TOL and U.rel_err(single, want) < F32_TOL
    else:
        assert U.bf16_close(whole, want) and U.bf16_close(single, want)
        assert U.bf16_close(whole, single, tol=3e-2)


@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 2], [5, 1, 17, 2, 40], [64, 2, 63], [1, 70, 2], [33, 33, 33, 33]])
def test_portions_of_several_sizes(sizes):
    """Portions cut anywhere: inside a page (8 tokens), a key tile (32) and a segment of the recurrence (64)."""
    cfg = U.config(**FULL)
    W = U.weights(cfg, seed=11)
    t = toks(140, seed=4)
    want = U.oracle_logits(cfg, W, t)
    assert U.rel_err(U.run_portions(cfg, W, t, sizes), want) < F32_TOL
    assert U.bf16_close(U.run_portions(cfg, W, t, sizes, "bfloat16"), want)


@pytest.mark.parametrize("heads,dim,vdim", [(2, 8, 16), (1, 24, 40), (2, 72, 100), (1, 128, 128)])
def test_long_recurrent_spans_run_as_segments_with_a_carry(heads, dim, vdim):
    """Spans above 64 tokens take the segment path (own contributions side by side, decay products, a carry, outputs): whole
    prompts and a long portion behind a short one against the oracle, and the state it leaves against decoding on."""
    cfg = U.config([(U.parallel(left_scale=0.3, r_heads=heads, r_dim=dim, r_vdim=vdim, tau=8.0), None)], width=24)
    W = U.weights(cfg, seed=13)
    t = toks(300, seed=5)
    want = U.oracle_logits(cfg, W, t)
    assert U.rel_err(U.run_whole(cfg, W, t), want) < F32_TOL
    assert U.rel_err(U.run_portions(cfg, W, t, [7, 200, 65, 20]), want) < F32_TOL


TENSOR_CORE_SHAPES = {
    # bfloat16 with dim % 8 == 0 and vdim % 16 == 0 runs attention on the tensor cores; the float32 run of the same model takes the
    # fp32-arithmetic kernel
    "sigmoid_16": [(U.attention(heads=4, kv_heads=2, dim=16, rot_dims=8), None)],
    "sigmoid_112_three_per_group": [(U.attention(heads=3, kv_heads=1, dim=112, rot_dims=112), None)],
    "softmax_dim8_vdim16": [(U.parallel(heads=4, kv_heads=4, dim=8, vdim=16, rot_dims=8, right_scale=0.2), None)],
    "softmax_dim24_vdim32_six_per_group": [(U.parallel(heads=6, kv_heads=1, dim=24, vdim=32, rot_dims=12, right_scale=0.2), None)],
    "softmax_dim72_vdim80": [(U.parallel(heads=2, kv_heads=1, dim=72, vdim=80, rot_dims=72, right_scale=0.2), None)],
    "softmax_dim128_vdim128_seventy_per_group": [(U.parallel(heads=70, kv_heads=1, dim=128, vdim=128, rot_dims=64, right_scale=0.2), None)],
}


@pytest.mark.parametrize("name", sorted(TENSOR_CORE_SHAPES))
def test_attention_on_tensor_cores(name):
    """Whole prompt, ragged portions (blocks that end inside a key tile) and decoding over a sliced history."""
    cfg = U.config(TENSOR_CORE_SHAPES[name], width=40)
    W = U.weights(cfg, seed=21)
    t = toks(330, seed=7)
    want = U.oracle_logits(cfg, W, t)
    assert U.rel_err(U.run_portions(cfg, W, t, [100, 3, 150, 64], page_size=16), want) < F32_TOL
    e16 = U.row_errs(U.run_whole(cfg, W, t, "bfloat16", page_size=16), want)
    assert float(np.quantile(e16, 0.8)) < 3e-2 and float(e16.max()) < 0.3
    e16 = U.row_errs(U.run_portions(cfg, W, t, [100, 3, 150, 64], "bfloat16", page_size=16), want)
    assert float(np.quantile(e16, 0.8)) < 3e-2 and float(e16.max()) < 0.3


def test_gated_linear_attention_with_heads_above_128():
    cfg = U.config([(U.parallel(left_scale=0.3, r_heads=1, r_dim=136, r_vdim=144, tau=8.0), None)], width=24)
    W = U.weights(cfg, seed=13)
    t = toks(100, seed=5)
    assert U.rel_err(U.run_portions(cfg, W, t, [70, 2, 20]), U.oracle_logits(cfg, W, t)) < F32_TOL


@pytest.mark.parametrize("width", [40, 300, 600, 1100])
def test_prompt_sized_passes_at_several_widths(width):
    """A prompt of 1100 tokens in one pass at four widths (rows shorter and longer than a block of the boundary kernel), through a
    looped layer (the [x ; x0] output).  Against the oracle in float32, and in bfloat16."""
    cfg = U.config([(U.parallel(heads=1, kv_heads=1, r_heads=1), U.dense(ff=16))], width=width, loop=(0, 1, 2))
    W = U.weights(cfg, seed=33)
    t = toks(1100, seed=14)
    want = U.oracle_logits(cfg, W, t)
    assert U.rel_err(U.run_whole(cfg, W, t, pool_tokens=1152, page_size=64), want) < F32_TOL
    assert U.bf16_close(U.run_whole(cfg, W, t, "bfloat16", pool_tokens=1152, page_size=64), want)


def test_persistent_products_agree_with_the_tiled_ones(monkeypatch):
    """A pass of 5120 prompt tokens is large enough for the persistent tensor-core products (plain: the input projection of a
    wide parallel layer; paired gate / up tiles with the gelu epilogue).  The same pass with DIS_STACK_PERSIST=0 takes the
    tiled products; both round the same operands to bfloat16, so the logits agree to accumulation order."""
    cfg = U.config([(U.parallel(heads=8, kv_heads=2, dim=64, vdim=64, rot_dims=32, r_heads=8, r_dim=64, r_vdim=64, rank=16), U.dense(ff=1024))],
                   width=128, vocab=64)
    W = U.weights(cfg, seed=27)
    seqs = [toks(640, vocab=64, seed=80 + i) for i in range(8)]
    res = []
    for flag in ("1", "0"):
        monkeypatch.setenv("DIS_STACK_PERSIST", flag)
        e = U.engine(cfg, W, "bfloat16", max_batch=8, pool_tokens=8 * 704, page_size=64, max_step_tokens=8 * 640, rows=64)
        P = InferenceParams(max_tokens=1 << 20, temperature=0.0)
        slots = [e.seq_add(sq, P) for sq in seqs]
        for sl in slots:
            e.seq_probe(sl, [5, 300, 638])
        e.step(slots)
        res.append(e.last_logits(e.last_logit_rows()).copy())
        e.close()
    assert res[0].shape == (8 * 4, 64)
    assert U.rel_err(res[0], res[1]) < 1e-3
    assert np.abs(res[0]).max() > 1e-2


def test_attention_over_slices_of_the_history():
    """A single decoding sequence with a long history has its keys cut into slices that a second kernel merges; both weight
    forms, in prompts and decoding, against the oracle."""
    cfg = U.config([(U.parallel(), None), (U.attention(), U.dense())], loop=(0, 2, 2))
    W = U.weights(cfg, seed=15)
    t = toks(700, seed=6)
    want = U.oracle_logits(cfg, W, t)
    for dtype in ("float32", "bfloat16"):
        e = U.engine(cfg, W, dtype, pool_tokens=768, page_size=64)
        f = U.Feeder(e)
        f.step([("a", t, 300)])
        f.step([("a", t, 5)])      # one query block, 305 keys: slices
        f.step([("a", t, 330)])
        for _ in range(65):
            f.step([("a", t, 1)])
        got = f.end("a")
        e.close()
        assert U.rel_err(got, want) < F32_TOL if dtype == "float32" else U.bf16_close(got, want)


def test_batches_of_unequal_requests_against_each_alone():
    cfg = U.config(**FULL)
    W = U.weights(cfg, seed=13)
    seqs = {k: toks(n, seed=20 + i) for i, (k, n) in enumerate([("a", 90), ("b", 33), ("c", 7), ("d", 58)])}
    want = {k: U.oracle_logits(cfg, W, v) for k, v in seqs.items()}
    e = U.engine(cfg, W, max_batch=4, pool_tokens=512)
    f = U.Feeder(e)
    f.step([("a", seqs["a"], 50), ("b", seqs["b"], 2)])
    f.step([("a", seqs["a"], 1), ("b", seqs["b"], 20), ("c", seqs["c"], 7)])
    f.step([("d", seqs["d"], 30), ("a", seqs["a"], 1), ("b", seqs["b"], 1)])
    while any(f.fed[k] < len(seqs[k]) for k in seqs):
        f.step([(k, seqs[k], min(3 if k == "d" else 1, len(seqs[k]) - f.fed[k])) for k in seqs if f.fed[k] < len(seqs[k])])
    for k in seqs:
        assert U.rel_err(f.end(k), want[k]) < F32_TOL, k
    e.close()


def test_pages_and_slots_are_freed_and_used_again():
    """Two slots and a pool of 12 pages: six sequences pass through them; the recurrent state and the cached keys and values
    of the sequence before (of every loop pass) must not reach the next one."""
    cfg = U.config(**FULL)
    W = U.weights(cfg, seed=17)
    e = U.engine(cfg, W, max_batch=2, pool_tokens=96, page_size=8)
    f = U.Feeder(e)
    lens = [40, 17, 48, 9, 33, 41]
    seqs = [toks(n, seed=40 + i) for i, n in enumerate(lens)]
    live = []
    for i, s in enumerate(seqs):
        if len(live) == 2:
            k = live.pop(0)
            while f.fed[k] < len(seqs[k]):
                f.step([(k, seqs[k], 1)] + [(o, seqs[o], 1) for o in live if f.fed[o] < len(seqs[o])])
            assert U.rel_err(f.end(k), U.oracle_logits(cfg, W, seqs[k])) < F32_TOL, k
        f.step([(i, s, len(s) - 5)] + [(o, seqs[o], 1) for o in live if f.fed[o] < len(seqs[o])])
        live.append(i)
    for k in live:
        while f.fed[k] < len(seqs[k]):
            f.step([(k, seqs[k], 1)])
        assert U.rel_err(f.end(k), U.oracle_logits(cfg, W, seqs[k])) < F32_TOL, k
    assert e.status().kv_pages_free == e.status().kv_pages_total
    e.close()


@pytest.mark.parametrize("decode_tail", [0, 40])
def test_far_keys_and_page_borders_with_peaked_weights(decode_tail):
    """A large score scale makes every softmax query put its weight on one key and every sigmoid weight 0 or 1, wherever in
    the 300 tokens the key lies: a key that is lost, shifted by one or read from the wrong page changes the output by its
    full size."""
    cfg = U.config([(U.parallel(scale=6.0, right_scale=0.05), None), (U.attention(scale=4.0), None)])
    W = U.weights(cfg, seed=19, gain=2.0)
    t = toks(300, seed=6)
    want = U.oracle_logits(cfg, W, t)
    e = U.engine(cfg, W, pool_tokens=320, page_size=16)
    f = U.Feeder(e)
    f.step([("a", t, 300 - decode_tail)])
    for _ in range(decode_tail):
        f.step([("a", t, 1)])
    got = f.end("a")
    e.close()
    assert U.rel_err(got, want) < 1e-4


def _planted(kind, n=8):
    """Hand-made weights for one layer of width n with one-hot token embeddings (layer norms keep a one-hot row's pattern):
    the query of token 2 points at the key of token 1 and at nothing else."""
    if kind == "softmax":
        cfg = U.config([(U.parallel(heads=1, kv_heads=1, dim=n, vdim=n, rot_dims=0, scale=1.0, right_scale=0.0, r_heads=1, r_dim=4, r_vdim=4,
                                    rank=2), None)], vocab=n, width=n, embed_scale=1.0, logit_scale=1.0)
        a = "l0.mix.left."
    else:
        cfg = U.config([(U.attention(heads=1, kv_heads=1, dim=n, rot_dims=0, scale=1.0), None)], vocab=n, width=n, embed_scale=1.0,
                       logit_scale=1.0)
        a = "l0.mix."
    W = U.weights(cfg, seed=23)
    eye = np.eye(n, dtype=np.float32)
    W["embed"] = eye.copy()
    W["l0.norm1"], W["l0.norm1.b"] = np.ones(n, np.float32), np.zeros(n, np.float32)
    q = np.zeros((n, n), np.float32)
    if kind == "softmax":
        # after the layer norm a one-hot row e_i is c (e_i - 1/n), c = sqrt(n^2 / (n - 1)); k = that row, q of token 2 = 16 e_1
        q[1, 2] = 16.0
        W[a + "q.norm"], W[a + "k.norm"] = np.full(n, 3.0, np.float32), np.ones(n, np.float32)
        W[a + "k"], W[a + "v"] = eye.copy(), eye.copy()
    else:
        q[1, 2] = 8.0
        W[a + "q.b"] = np.zeros(n, np.float32)
        W[a + "k.b"] = np.zeros(n, np.float32)
        W[a + "k"] = eye.copy()
        W[a + "temp"], W[a + "pb"] = np.ones(1, np.float32), np.full(1, -30.0, np.float32)
    W[a + "q"] = q
    return cfg, W


@pytest.mark.parametrize("kind,n,dtype", [("softmax", 8, "float32"), ("sigmoid", 8, "float32"), ("softmax", 16, "bfloat16"), ("sigmoid", 16, "bfloat16")])
def test_a_key_planted_far_back_is_found(kind, n, dtype):
    """Token 1 occurs once among 260 tokens; the last token (2) looks for it.  With sigmoid weights under a bias of -30 only
    that key gets a weight at all; with softmax it takes nearly all of it.  The output at the last position then changes with
    the planted key, wherever it stands: next to a page border on either side, at the very start, or just before the query."""
    cfg, W = _planted(kind, n)
    base = [int(x) for x in np.random.default_rng(1).integers(3, n, 260)]
    base[-1] = 2
    without = U.oracle_logits(cfg, W, base)[-1]
    for where in (0, 31, 32, 63, 64, 127, 128, 191, 192, 258):
        t = list(base)
        t[where] = 1
        want = U.oracle_logits(cfg, W, t)
        assert np.abs(want[-1] - without).max() > 0.05  # the planted key decides the output
        for tail in (0, 3):  # the query inside a prompt portion, and decoded alone
            e = U.engine(cfg, W, dtype, pool_tokens=320, page_size=64)
            f = U.Feeder(e)
            f.step([("a", t, 260 - tail)])
            for _ in range(tail):
                f.step([("a", t, 1)])
            got = f.end("a")
            e.close()
            assert U.rel_err(got, want) < (1e-4 if dtype == "float32" else 2e-2), (where, tail)


def test_sigmoid_bias_and_temperature_per_head():
    cfg = U.config([(U.attention(heads=4, kv_heads=2), None)])
    W = U.weights(cfg, seed=29)
    t = toks(30, seed=8)
    res = []
    for pb, temp in ((-6.0, 1.0), (0.5, 1.0), (0.5, 3.0)):
        W["l0.mix.pb"] = np.asarray([pb, 0.0, pb, -1.0], np.float32)
        W["l0.mix.temp"] = np.asarray([temp, 1.0, 0.25, temp], np.float32)
        want = U.oracle_logits(cfg, W, t)
        assert U.rel_err(U.run_whole(cfg, W, t), want) < F32_TOL
        res.append(want)
    assert np.abs(res[0] - res[1]).max() > 1e-2 and np.abs(res[1] - res[2]).max() > 1e-2


def test_first_tokens_of_a_sequence():
    cfg = U.config(**FULL)
    W = U.weights(cfg, seed=31)
    for n in (1, 2, 3, 5):
        t = toks(n, seed=50 + n)
        assert U.rel_err(U.run_whole(cfg, W, t), U.oracle_logits(cfg, W, t)) < F32_TOL, n
    t = toks(9, seed=60)
    assert U.rel_err(U.run_portions(cfg, W, t, [1, 1, 2, 1, 4]), U.oracle_logits(cfg, W, t)) < F32_TOL


def test_long_decoding_keeps_state_and_cache_exact():
    cfg = U.config([(U.parallel(tau=64.0), U.dense()), (U.attention(), None)], loop=(0, 1, 2))
    W = U.weights(cfg, seed=37)
    t = toks(420, seed=9)
    want = U.oracle_logits(cfg, W, t)
    e = U.engine(cfg, W, pool_tokens=448, page_size=64)
    f = U.Feeder(e)
    f.step([("a", t, 20)])
    for _ in range(400):
        f.step([("a", t, 1)])
    got = f.end("a")
    e.close()
    assert U.rel_err(got, want) < 5e-5


ODD = [(U.parallel(heads=6, kv_heads=3, dim=10, vdim=14, rot_dims=10, r_heads=2, r_dim=36, r_vdim=20, tau=2.0, rank=3, left_scale=1.3, right_scale=0.4),
        U.dense(ff=20)),
       (U.attention(heads=5, kv_heads=5, dim=6, rot_dims=2, scaling=(2.0, 0.5, 8.0, 100)), None),
       (U.parallel(heads=1, kv_heads=1, dim=40, vdim=8, rot_dims=0, r_heads=5, r_dim=4, r_vdim=68, tau=30.0, rank=9), U.dense(ff=36)),
       (U.attention(heads=8, kv_heads=2, dim=20, rot_dims=20, base=77.0), U.dense(ff=8))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,vocab,loop", [(72, 131, (0, 2, 3)), (136, 61, (2, 4, 2)), (50, 33, None)])
def test_other_sizes(dtype, width, vocab, loop):
    cfg = U.config(ODD, vocab=vocab, width=width, eps=1e-3, loop=loop, embed_scale=0.7, logit_scale=1.9)
    W = U.weights(cfg, seed=41)
    t = toks(75, vocab=vocab, seed=10)
    want = U.oracle_logits(cfg, W, t)
    got = U.run_portions(cfg, W, t, [33, 2, 1, 1, 30, 8], dtype, page_size=16, pool_tokens=128)
    assert U.rel_err(got, want) < F32_TOL if dtype == "float32" else U.bf16_close(got, want)


def test_model_folder_round_trip(tmp_path):
    """config.json + model.safetensors written by the test, read back through the registry (the rank of the decay projection
    comes from a tensor's shape), loaded and run."""
    import json
    import struct
    cfg = U.config(**FULL)
    for ly in cfg["layers"]:
        if ly["type"] == "parallel":
            del ly["mixer"]["right"]["rank"]
    W = U.weights(U.config(**FULL), seed=43)
    header, blobs, at = {}, [], 0
    for name, a in W.items():
        bits = (np.ascontiguousarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [at, at + len(bits)]}
        blobs.append(bits)
        at += len(bits)
    hj = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    t = toks(20, seed=12)
    e = models.load_model(str(tmp_path), dtype="float32", max_batch=2, max_tokens=64, page_size=16, max_step_tokens=64, max_logit_rows=68)
    f = U.Feeder(e)
    f.step([("a", t, 20)])
    got = f.end("a")
    e.close()
    assert U.rel_err(got, U.oracle_logits(U.config(**FULL), W, t)) < F32_TOL


def test_greedy_generation_through_the_scheduler():
    """Requests of unequal length through the admission queue and the continuous batcher; greedy tokens equal the oracle's,
    except where the oracle's top two logits are closer than float32 noise."""
    cfg = U.config(vocab=40, **FULL)
    W = U.weights(cfg, seed=43)
    e = U.engine(cfg, W, max_batch=3, pool_tokens=256, page_size=8, max_step_tokens=64)
    cb = ContinuousBatcher(e, max_active=3)
    cb.set_prefill_budget(16)  # prompts are read in portions beside the running sequences
    prompts = [toks(n, vocab=40, seed=70 + n) for n in (5, 37, 12, 1, 26)]
    new = [9, 6, 12, 7, 5]
    for i, p in enumerate(prompts):
        cb.submit(i, p, InferenceParams(new[i], 0.0))
    res = cb.run_until_idle()
    for i, p in enumerate(prompts):
        seq = list(p)
        got = res[i]["tokens"]
        assert len(got) == new[i]
        for j in range(new[i]):
            lg = U.oracle_logits(cfg, W, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if int(np.argmax(lg)) != got[j]:
                assert top2[1] - top2[0] < 1e-4, (i, j)
            seq.append(got[j])
    cb.close()
    e.close()
