"""The layer-list decoder family (Kidolorn) against the plain oracle in tests/kidolorn_oracle.py: every mechanism alone,
whole prompts against token-by-token decoding, portions of many sizes, unequal batches, reuse of pages and state slots,
far keys and page borders, the first tokens, long decoding, odd sizes, and greedy generation through the scheduler."""
import numpy as np
import pytest

from distributed_inference_server_b200 import ContinuousBatcher, InferenceParams
from distributed_inference_server_b200 import binding as B
from tests import _stack_util as U

pytestmark = pytest.mark.gpu
F32_TOL = 2e-4   # float32 engine against the float64 oracle (these narrow random models are not well conditioned everywhere)
SAME = 4e-6      # two float32 schedules of the same tokens against each other


def toks(n, vocab=50, seed=0):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


MECHANISMS = {
    "lightning": [(U.lightning(), None)],
    "lightning_one_head": [(U.lightning(heads=1, dim=12, vdim=20, decay=[0.97]), None)],
    "mingru": [(U.mingru(), None)],
    "latent": [(U.latent(), None)],
    "latent_partial_rotation": [(U.latent(heads=3, dim=12, rot_dim=8, vdim=10, kv_rank=20, rot_dims=4, base=100.0), None)],
    "latent_rows_of_16_bytes": [(U.latent(heads=2, dim=8, rot_dim=8, vdim=12, kv_rank=24), None)],
    "latent_shared": [(U.latent(), None), (U.mingru(), None), (U.latent(kv_from=0, vdim=20, dim=4, heads=3), None)],
    "dense": [(U.mingru(8), U.dense())],
    "moe": [(U.mingru(8), U.moe())],
    "moe_top_all": [(U.mingru(8), U.moe(experts=3, top=3))],
    "moe_top_one": [(U.mingru(8), U.moe(experts=5, top=1))],
}


@pytest.mark.parametrize("name", sorted(MECHANISMS))
@pytest.mark.parametrize("taps", [0, 1, 3])
def test_each_mechanism_alone(name, taps):
    cfg = U.config(MECHANISMS[name], taps=taps)
    W = U.weights(cfg, seed=3)
    t = toks(70, seed=1)
    want = U.oracle_logits(cfg, W, t)
    got = U.run_whole(cfg, W, t)
    assert U.rel_err(got, want) < F32_TOL
    got16 = U.run_whole(cfg, W, t, dtype="bfloat16")
    assert U.bf16_close(got16, want)


def test_residual_stream_after_every_layer_matches():
    """One layer more changes only what follows it: prefixes of the layer list reproduce the oracle's stream layer by layer
    (through the logits of a model cut after each layer)."""
    layers = [(U.lightning(), U.dense()), (U.latent(), U.moe()), (U.latent(kv_from=1), U.dense()), (U.mingru(), U.moe())]
    t = toks(40, seed=2)
    for n in range(1, len(layers) + 1):
        cfg = U.config(layers[:n])
        W = U.weights(cfg, seed=5)
        assert U.rel_err(U.run_whole(cfg, W, t), U.oracle_logits(cfg, W, t)) < F32_TOL, n


FULL = [(U.mingru(), U.moe()), (U.latent(), U.dense()), (U.lightning(), U.moe()), (U.latent(kv_from=1), None),
        (U.latent(heads=1, dim=16, rot_dim=8, vdim=8, kv_rank=8), U.dense())]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_against_token_by_token_decoding(dtype):
    cfg = U.config(FULL)
    W = U.weights(cfg, seed=7)
    t = toks(60, seed=3)
    want = U.oracle_logits(cfg, W, t)
    e = U.engine(cfg, W, dtype)
    f = U.Feeder(e)
    f.step([("w", t, len(t))])
    for _ in t:
        f.step([("d", t, 1)])
    whole, single = f.end("w"), f.end("d")
    e.close()
    if dtype == "float32":
        assert U.rel_err(whole, want) < F32_TOL and U.rel_err(single, want) < F32_TOL
        assert U.rel_err(single, whole) < SAME
    else:
        assert U.bf16_close(whole, want) and U.bf16_close(single, want)
        assert U.rel_err(single, whole) < 2e-2  # the same roundings in both schedules up to the order of sums


@pytest.mark.parametrize("sizes", [[2] * 40, [3, 2, 7, 1, 16, 9, 2, 8, 1, 1, 30], [1, 79], [64, 16], [5, 8, 8, 8, 51]])
def test_portions_of_several_sizes(sizes):
    """Portions cut in the middle of pages (8 tokens here) and of the convolution's reach, down to two tokens."""
    cfg = U.config(FULL, taps=4)
    W = U.weights(cfg, seed=11)
    t = toks(sum(sizes), seed=4)
    want = U.oracle_logits(cfg, W, t)
    e = U.engine(cfg, W)
    f = U.Feeder(e)
    for n in sizes:
        f.step([("a", t, n)])
    got = f.end("a")
    e.close()
    assert U.rel_err(got, want) < F32_TOL
    assert U.rel_err(got, U.run_whole(cfg, W, t)) < SAME


@pytest.mark.parametrize("heads,dim,vdim", [(2, 8, 16), (1, 72, 40), (3, 128, 128), (1, 136, 144)])
def test_long_recurrent_spans_run_as_segments_with_a_carry(heads, dim, vdim):
    """A span longer than a segment (64 tokens) of the decayed linear-attention scan, or of the gated recurrence, is cut into
    segments that run side by side and are joined by a carry pass.  Spans of one token, of exactly one or two segments, with a
    ragged last segment and with a start in the middle of a sequence share passes here; all must agree with the oracle and
    with token-by-token feeding.  The last size is beyond what the register kernel holds (128 x 128 per head) and runs on the
    kernel that keeps the state in shared memory."""
    cfg = U.config([(U.lightning(heads=heads, dim=dim, vdim=vdim, decay=[0.999, 0.93, 0.5][:heads]), None), (U.mingru(24), None)],
                   width=40)
    W = U.weights(cfg, seed=61)
    a, b, c = toks(300, seed=41), toks(140, seed=42), toks(129, seed=43)
    wa, wb, wc = (U.oracle_logits(cfg, W, t) for t in (a, b, c))
    e = U.engine(cfg, W, pool_tokens=640, page_size=16)
    f = U.Feeder(e)
    f.step([("a", a, 130), ("b", b, 1), ("c", c, 64)])
    f.step([("a", a, 1), ("b", b, 128), ("c", c, 65)])
    f.step([("a", a, 169), ("b", b, 11)])
    ga, gb, gc = f.end("a"), f.end("b"), f.end("c")
    for _ in c:
        f.step([("s", c, 1)])
    gs = f.end("s")
    e.close()
    assert max(U.rel_err(ga, wa), U.rel_err(gb, wb), U.rel_err(gc, wc)) < F32_TOL
    assert U.rel_err(gs, gc) < 1e-5


def test_few_rows_product_agrees_with_the_tiled_one():
    """Passes of at most 64 rows take the product kernel that streams the weights once (experts with a few tokens, decode);
    larger passes the tiled one.  The same tokens fed both ways must give the same logits."""
    cfg = U.config([(U.latent(heads=2, dim=8, rot_dim=8, vdim=16, kv_rank=24), U.moe(ff=16, experts=4, top=2)),
                    (U.mingru(32), U.dense(ff=40))], width=32)
    W = U.weights(cfg, seed=67)
    t = toks(100, seed=44)
    want = U.oracle_logits(cfg, W, t)
    whole = U.run_whole(cfg, W, t)
    e = U.engine(cfg, W)
    f = U.Feeder(e)
    for n in [30, 9, 1, 1, 40, 19]:
        f.step([("a", t, n)])
    got = f.end("a")
    e.close()
    assert U.rel_err(whole, want) < F32_TOL and U.rel_err(got, want) < F32_TOL
    assert U.rel_err(got, whole) < 1e-5


def test_long_portions_in_bfloat16_take_the_matrix_product_path():
    """In bfloat16, latent attention of portions of 32 tokens or more runs as tensor-core products over latents gathered out of
    their pages (kv_rank and kv_rank + rot_dim multiples of 8); shorter portions and single tokens run on the paged kernel.
    Both must agree with the oracle, also when one sequence changes between them and when two sequences share a pass."""
    cfg = U.config([(U.latent(heads=2, dim=8, rot_dim=8, vdim=16, kv_rank=24), U.dense()),
                    (U.latent(heads=4, dim=16, rot_dim=8, vdim=8, kv_rank=24, kv_from=0), None)], width=64)
    W = U.weights(cfg, seed=47)
    a, b = toks(150, seed=31), toks(90, seed=32)
    wa, wb = U.oracle_logits(cfg, W, a), U.oracle_logits(cfg, W, b)
    e = U.engine(cfg, W, "bfloat16", pool_tokens=320, page_size=16)
    f = U.Feeder(e)
    f.step([("a", a, 40), ("b", b, 5)])
    f.step([("a", a, 3), ("b", b, 64)])
    f.step([("a", a, 64), ("b", b, 1)])
    f.step([("a", a, 1), ("b", b, 20)])
    f.step([("a", a, 42)])
    ga, gb = f.end("a"), f.end("b")
    e.close()
    assert U.bf16_close(ga, wa) and U.bf16_close(gb, wb)
    assert float(np.median(U.row_errs(ga, wa))) < 2e-2


@pytest.mark.parametrize("heads", [1, 2, 5, 16])
def test_short_portions_and_decoding_in_bfloat16_on_the_tensor_core_attention_kernel(heads):
    """bfloat16 with kv_rank a multiple of 8 and kv_rank + rot_dim a multiple of 16: portions below 32 tokens and single tokens
    run latent attention with the (token, head) pairs as the rows of tensor-core tiles over 64 latents at a time; beyond 256
    tokens of history the history is cut into slices that a merge kernel joins.  Query blocks of several tokens (few heads),
    of one token (16 heads), ragged last tiles, and a second sequence in the same passes."""
    cfg = U.config([(U.latent(heads=heads, dim=8, rot_dim=8, vdim=8, kv_rank=40), U.dense()),
                    (U.latent(heads=3, dim=8, rot_dim=8, vdim=16, kv_rank=40, kv_from=0), None)], width=64)
    W = U.weights(cfg, seed=71)
    a, b = toks(345, seed=51), toks(100, seed=52)
    wa, wb = U.oracle_logits(cfg, W, a), U.oracle_logits(cfg, W, b)
    e = U.engine(cfg, W, "bfloat16", pool_tokens=512, page_size=16)
    f = U.Feeder(e)
    f.step([("a", a, 21), ("b", b, 1)])
    f.step([("a", a, 31), ("b", b, 30)])
    f.step([("a", a, 230), ("b", b, 9)])       # a: the matrix-product path; b: short
    for _ in range(30):                        # a decodes past 256 tokens of history (sliced), b stays below
        f.step([("a", a, 1), ("b", b, 2)])
    f.step([("a", a, 33)])
    ga, gb = f.end("a"), f.end("b")
    e.close()
    assert U.bf16_close(ga, wa) and U.bf16_close(gb, wb)
    assert float(np.median(U.row_errs(ga, wa))) < 2e-2 and float(np.median(U.row_errs(gb, wb))) < 2e-2


@pytest.mark.parametrize("big", [False, True])
def test_passes_of_256_tokens_in_bfloat16_run_the_head_products_on_tensor_cores(big):
    """From 256 tokens in a pass, the query absorption and the value expansion of latent attention run as one tensor-core
    product per head over that head's rows packed together (bfloat16; dim, kv_rank and kv_rank + rot_dim multiples of 8).
    A pass above and one below that size, two sequences in one pass, against the oracle and against each other."""
    if big:  # more than one 64-wide K block and more than one 128-row weight tile in every product
        cfg = U.config([(U.latent(heads=4, dim=72, rot_dim=32, vdim=136, kv_rank=160), U.dense(ff=96)),
                        (U.latent(heads=2, dim=136, rot_dim=32, vdim=64, kv_rank=160, kv_from=0), None)], width=192)
    else:
        cfg = U.config([(U.latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40), U.dense()),
                        (U.latent(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=40, kv_from=0), None)], width=64)
    W = U.weights(cfg, seed=53)
    a, b = toks(330, seed=33), toks(120, seed=34)
    wa, wb = U.oracle_logits(cfg, W, a), U.oracle_logits(cfg, W, b)
    e = U.engine(cfg, W, "bfloat16", pool_tokens=512, page_size=16)
    f = U.Feeder(e)
    f.step([("a", a, 280), ("b", b, 70)])
    f.step([("a", a, 50), ("b", b, 50)])
    ga, gb = f.end("a"), f.end("b")
    f.step([("c", a, 200)])
    f.step([("c", a, 130)])
    gc = f.end("c")
    e.close()
    assert U.bf16_close(ga, wa) and U.bf16_close(gb, wb) and U.bf16_close(gc, wa)
    assert float(np.median(U.row_errs(ga, wa))) < 2e-2 and float(np.median(U.row_errs(ga, gc))) < 2e-2


@pytest.mark.parametrize("experts,top", [(2, 1), (4, 2), (3, 3)])
def test_large_expert_passes_in_bfloat16_run_one_product_per_expert(experts, top):
    """A pass with at least 64 rows per expert on average sorts its rows by expert and runs each expert's rows as one
    tensor-core product; smaller passes (the single tokens after the prompt) use the grouped fp32-FMA product."""
    cfg = U.config([(U.mingru(16), U.moe(ff=16, experts=experts, top=top)), (U.lightning(), U.moe(ff=24, experts=experts, top=top))])
    W = U.weights(cfg, seed=53)
    t = toks(260, seed=33)
    want = U.oracle_logits(cfg, W, t)
    e = U.engine(cfg, W, "bfloat16", pool_tokens=320, page_size=64)
    f = U.Feeder(e)
    f.step([("a", t, 250)])
    for _ in range(10):
        f.step([("a", t, 1)])
    got = f.end("a")
    e.close()
    assert U.bf16_close(got, want)
    assert float(np.median(U.row_errs(got, want))) < 2e-2


def test_batches_of_unequal_requests_against_each_alone():
    cfg = U.config(FULL)
    W = U.weights(cfg, seed=13)
    seqs = {k: toks(n, seed=20 + i) for i, (k, n) in enumerate([("a", 90), ("b", 33), ("c", 7), ("d", 58)])}
    want = {k: U.oracle_logits(cfg, W, v) for k, v in seqs.items()}
    e = U.engine(cfg, W, max_batch=4, pool_tokens=512)
    f = U.Feeder(e)
    # portions of some beside single tokens of others
    f.step([("a", seqs["a"], 50), ("b", seqs["b"], 2)])
    f.step([("a", seqs["a"], 1), ("b", seqs["b"], 20), ("c", seqs["c"], 7)])
    f.step([("d", seqs["d"], 30), ("a", seqs["a"], 1), ("b", seqs["b"], 1)])
    while any(f.fed[k] < len(seqs[k]) for k in seqs):
        f.step([(k, seqs[k], min(3 if k == "d" else 1, len(seqs[k]) - f.fed[k])) for k in seqs if f.fed[k] < len(seqs[k])])
    for k in seqs:
        assert U.rel_err(f.end(k), want[k]) < F32_TOL, k
    e.close()


def test_pages_and_slots_are_freed_and_used_again():
    """Two slots and a pool of 12 pages: six sequences pass through them; a slot's recurrent state, convolution tail and
    pages of the sequence before must not reach the next one."""
    cfg = U.config(FULL)
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
def test_far_keys_and_page_borders_with_a_peaked_softmax(decode_tail):
    """A large score scale and strongly negative sinks make every query put its weight on one key, wherever in the 300
    tokens it lies: a key that is lost, shifted by one, or read from the wrong page changes the output by its full size."""
    cfg = U.config([(U.latent(heads=2, dim=8, rot_dim=4, vdim=12, kv_rank=16, scale=6.0), None),
                    (U.latent(kv_from=0, heads=2, dim=8, rot_dim=4, vdim=12, kv_rank=16, scale=6.0), None)], taps=0)
    W = U.weights(cfg, seed=19, gain=2.0)
    for k in W:
        if k.endswith("sink"):
            W[k] = np.full_like(W[k], -30.0)
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


def test_a_key_planted_far_back_is_found():
    """Hand-made weights: tokens are one-hot, the latent is the token itself, and the query of token 2 points at the key of
    token 1 with a score of 24 while every other score is 0.  Token 1 occurs once among 260 tokens; the output at the last
    position (token 2) is then token 1's value, wherever it stands: next to a page border on either side, at the very
    start, or just before the query."""
    n = 8
    cfg = U.config([(U.latent(heads=1, dim=n, rot_dim=0, vdim=n, kv_rank=n, scale=1.0), None)], taps=0, vocab=n, width=n)
    W = U.weights(cfg, seed=23)
    eye = np.eye(n, dtype=np.float32)
    W["embed"] = eye * np.float32(np.sqrt(n))
    W["l0.norm1"] = np.asarray(1.0, np.float32)
    W["l0.mix.dkv"], W["l0.mix.dkv.norm"], W["l0.mix.uk"] = eye.copy(), np.ones(n, np.float32), eye.copy()
    q = np.zeros((n, n), np.float32)
    q[1, 2] = 3.0
    W["l0.mix.q"] = q
    W["l0.mix.sink"] = np.full((1,), -40.0, np.float32)
    base = [int(x) for x in np.random.default_rng(1).integers(3, n, 260)]
    base[-1] = 2
    without = U.oracle_logits(cfg, W, base)[-1]
    for where in (0, 63, 64, 127, 128, 191, 192, 258):
        t = list(base)
        t[where] = 1
        want = U.oracle_logits(cfg, W, t)
        assert np.abs(want[-1] - without).max() > 0.05  # the planted key decides the output
        for tail in (0, 3):  # the query inside a prompt portion, and decoded alone
            e = U.engine(cfg, W, pool_tokens=320, page_size=64)
            f = U.Feeder(e)
            f.step([("a", t, 260 - tail)])
            for _ in range(tail):
                f.step([("a", t, 1)])
            got = f.end("a")
            e.close()
            assert U.rel_err(got, want) < 1e-4, (where, tail)


def test_sink_takes_weight_from_the_keys():
    cfg = U.config([(U.latent(), None)], taps=0)
    W = U.weights(cfg, seed=29)
    t = toks(30, seed=8)
    res = []
    for sink in (-20.0, 6.0):
        W["l0.mix.sink"] = np.full_like(W["l0.mix.sink"], sink)
        want = U.oracle_logits(cfg, W, t)
        assert U.rel_err(U.run_whole(cfg, W, t), want) < F32_TOL
        res.append(want)
    assert np.abs(res[0] - res[1]).max() > 1e-2


def test_first_tokens_of_a_sequence():
    """Positions 0 .. taps read zeros in front of the sequence; one-token prompts and one-token first portions."""
    cfg = U.config(FULL, taps=4)
    W = U.weights(cfg, seed=31)
    for n in (1, 2, 3, 5):
        t = toks(n, seed=50 + n)
        assert U.rel_err(U.run_whole(cfg, W, t), U.oracle_logits(cfg, W, t)) < F32_TOL, n
    t = toks(9, seed=60)
    e = U.engine(cfg, W)
    f = U.Feeder(e)
    for n in (1, 1, 2, 1, 4):
        f.step([("a", t, n)])
    assert U.rel_err(f.end("a"), U.oracle_logits(cfg, W, t)) < F32_TOL
    e.close()


def test_long_decoding_keeps_the_recurrent_state_exact():
    cfg = U.config([(U.lightning(heads=2, dim=8, vdim=8, decay=[0.999, 0.9]), None), (U.mingru(16), U.dense()), (U.latent(), None)])
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


ODD = [(U.latent(heads=3, dim=12, rot_dim=6, vdim=10, kv_rank=20, rot_dims=6), U.moe(ff=20, experts=3, top=2, limit=0.7)),
       (U.lightning(heads=3, dim=4, vdim=20, decay=[1.0, 0.5, 0.25]), None),
       (U.mingru(40), U.dense(ff=36, limit=0.5)),
       (U.latent(heads=3, dim=12, rot_dim=6, vdim=14, kv_rank=20, kv_from=0, scale=0.4), U.dense(ff=8, limit=3.0)),
       (U.latent(heads=5, dim=4, rot_dim=2, vdim=6, kv_rank=36), U.moe(ff=8, experts=6, top=6))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,vocab,taps", [(72, 131, 2), (136, 61, 5)])
def test_other_sizes(dtype, width, vocab, taps):
    cfg = U.config(ODD, vocab=vocab, width=width, taps=taps, eps=1e-3)
    W = U.weights(cfg, seed=41)
    t = toks(75, vocab=vocab, seed=10)
    want = U.oracle_logits(cfg, W, t)
    e = U.engine(cfg, W, dtype, page_size=16, pool_tokens=128)
    f = U.Feeder(e)
    for n in (33, 2, 1, 1, 30, 8):
        f.step([("a", t, n)])
    got = f.end("a")
    e.close()
    assert U.rel_err(got, want) < F32_TOL if dtype == "float32" else U.bf16_close(got, want)


def test_greedy_generation_through_the_scheduler():
    """Requests of unequal length through the admission queue and the continuous batcher; greedy tokens equal the oracle's,
    except where the oracle's top two logits are closer than float32 noise."""
    cfg = U.config(FULL, vocab=40)
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
