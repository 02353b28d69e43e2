"""Nagilix through the engine against the plain oracle (oracle/nagilix_oracle.py): each mechanism alone, prefill against
token-by-token decoding, portions down to two tokens, unequal batches, pages and slots used again, the edges of the
chunks made visible by a planted query/key pair, far keys and far tokens in the recurrent states, the carried inputs of
the convolutions across cuts, other sizes (also the degenerate ones), long decoding, and greedy generation through the
engine's own submit / scheduler / sampling path.  Configurations and weights are made here; nothing is read from disk
but what the test wrote."""
import numpy as np
import pytest

from nagilix_util import (feed_portions, feed_whole, left, make_config, mamba, moe, open_engine, oracle_for, parallel, plant_pair, random_weights,
                          rel_err, right, write_model_dir)

pytestmark = pytest.mark.gpu

F32_TOL = 2e-5     # fp32 engine vs float64 oracle, relative RMS over the vocabulary


def close32(got, want, scale=1.0):
    r = rel_err(got, want)
    assert np.median(r) < F32_TOL * scale, np.median(r)
    assert r.max() < 15 * F32_TOL * scale, (int(np.argmax(r)), r.max())


def close16(got, want):
    """bf16 serving precision on these tiny widths: a few percent per row; a row where rounding flips a close routing
    choice may be far off, so the bound is on the median and on the 90th percentile."""
    r = rel_err(got, want)
    assert np.median(r) < 0.06, np.median(r)
    assert np.quantile(r, 0.9) < 0.2, np.quantile(r, 0.9)


def toks(n, vocab, seed=0):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def build(tmp_path, layers, seed=0, wkw=None, **kw):
    cfg = make_config(layers, **kw)
    W = random_weights(cfg, seed=seed, **(wkw or {}))
    return cfg, W, write_model_dir(tmp_path / "m", cfg, W)


# both kinds of layers, with and without a feed-forward, chunks that are no multiple of a page
MIX = [parallel(), mamba(mlp=None),
       parallel(l=left(heads=3, kv_heads=3, dim=6, chunk=9, rot_dims=4, conv=2), r=right(heads=3, dim=4, vdim=6, rot_dims=2), mlp=None),
       mamba(inner=12, state=9, dt_rank=2, conv=2, mlp=moe(experts=4, identity=1, top=1))]


@pytest.fixture(scope="module")
def mix(tmp_path_factory):
    cfg, W, d = build(tmp_path_factory.mktemp("mix"), MIX)
    return cfg, W, d, oracle_for(cfg, W)


@pytest.fixture(scope="module")
def mix_wide(tmp_path_factory):
    """Chunks longer than any test sequence: a sequence holds all its pages, so a small pool really fills."""
    layers = [parallel(l=left(chunk=500))] + MIX[1:2] + [parallel(l=left(heads=2, kv_heads=1, chunk=0), mlp=None)]
    cfg, W, d = build(tmp_path_factory.mktemp("mixw"), layers, seed=5)
    return cfg, W, d, oracle_for(cfg, W)


# ---------------------------------------------------------------- each mechanism alone
LEFT, RIGHT = dict(left_only=True), dict(right_only=True)


@pytest.mark.parametrize("name,layers,kw,wkw", [
    ("left_only", [parallel(mlp=None)], {}, LEFT),
    ("left_full_heads_plain_causal", [parallel(l=left(heads=3, kv_heads=3, chunk=0), mlp=None)], {}, LEFT),
    ("left_one_kv_head", [parallel(l=left(heads=4, kv_heads=1, dim=4), mlp=None)], {}, LEFT),
    ("left_partial_rotation", [parallel(l=left(dim=10, rot_dims=4), mlp=None)], {}, LEFT),
    ("left_no_rotation", [parallel(l=left(rot_dims=0), mlp=None)], {}, LEFT),
    ("left_no_convolution", [parallel(l=left(conv=0), mlp=None)], {}, LEFT),
    ("left_two_taps", [parallel(l=left(conv=2), mlp=None)], {}, LEFT),
    ("left_six_taps", [parallel(l=left(conv=6), mlp=None)], {}, LEFT),
    ("left_chunk_of_one", [parallel(l=left(chunk=1), mlp=None)], {}, LEFT),
    ("left_chunk_of_a_page", [parallel(l=left(chunk=16), mlp=None)], {}, LEFT),
    ("left_odd_head_size", [parallel(l=left(dim=7, rot_dims=6), mlp=None)], {}, LEFT),
    ("right_only", [parallel(mlp=None)], {}, RIGHT),
    ("right_one_head_wide_value", [parallel(r=right(heads=1, dim=4, vdim=20, decay=[0.9]), mlp=None)], {}, RIGHT),
    ("right_many_rows", [parallel(r=right(heads=2, dim=40, vdim=8), mlp=None)], {}, RIGHT),
    ("right_partial_rotation", [parallel(r=right(dim=10, rot_dims=6), mlp=None)], {}, RIGHT),
    ("right_no_rotation", [parallel(r=right(rot_dims=0), mlp=None)], {}, RIGHT),
    ("both_branches", [parallel(mlp=None)], {}, {}),
    ("mamba_only", [mamba(mlp=None)], {}, {}),
    ("mamba_one_state", [mamba(inner=7, state=1, dt_rank=1, conv=2, mlp=None)], {}, {}),
    ("mamba_wide_state", [mamba(inner=9, state=40, dt_rank=4, conv=3, mlp=None)], {}, {}),
    ("mamba_sixteen_states", [mamba(inner=33, state=16, dt_rank=5, conv=4, mlp=None)], {}, {}),
    ("mamba_one_tap", [mamba(conv=1, mlp=None)], {}, {}),
    ("moe_with_identity", [parallel()], {}, {}),
    ("moe_without_identity", [parallel(mlp=moe(identity=0))], {}, {}),
    ("moe_top1", [mamba(mlp=moe(top=1))], {}, {}),
    ("moe_all_outputs_chosen", [parallel(mlp=moe(experts=3, identity=1, top=4))], {}, {}),
    ("moe_mostly_identity", [parallel(mlp=moe(experts=1, identity=3, top=2))], {}, {}),
    ("moe_tight_limit", [parallel(mlp=moe(limit=0.2))], {}, {}),
    ("one_stream", [parallel(), mamba()], dict(streams=1), {}),
    ("plain_residual", [parallel(), mamba()], dict(streams=None), {}),
    ("three_streams", [mamba(), parallel(mlp=None)], dict(streams=3), {}),
    ("ungated_write_back", [parallel(), mamba()], {}, dict(gated=False)),
    ("odd_width", [parallel(), mamba()], dict(width=21, vocab=33), {}),
    ("large_eps_in_every_norm", [parallel(), mamba()], dict(eps=0.05), {}),
    ("unit_logit_scale", [mamba(), parallel()], dict(logit_scale=1.0), {}),
])
def test_each_mechanism_matches_the_oracle(tmp_path, name, layers, kw, wkw):
    cfg, W, d = build(tmp_path, layers, seed=3, wkw=wkw, **kw)
    o = oracle_for(cfg, W)
    t = toks(29, cfg["vocab"], 1)
    want, layers_want = o.forward(t, return_layers=True)
    with open_engine(d) as e:
        e.debug_residuals(True)
        got = feed_whole(e, t)
        res = e.read_residuals().reshape(layers_want.shape)
    assert np.abs(res - layers_want).max() < 1e-4 * max(1.0, np.abs(layers_want).max()), name
    close32(got, want)


def test_bfloat16_serving_precision_stays_near_the_oracle(tmp_path):
    """Without routing decisions (every router output chosen) bf16 rounding moves every row by a few percent at most."""
    layers = [parallel(mlp=moe(experts=3, identity=1, top=4)), mamba(mlp=None), MIX[2], mamba(inner=16, state=8, mlp=moe(experts=2, identity=0, top=2))]
    cfg, W, d = build(tmp_path, layers, seed=9)
    t = toks(70, cfg["vocab"], 2)
    want, streams = oracle_for(cfg, W).forward(t, return_layers=True)
    with open_engine(d, dtype="bfloat16") as e:
        got = feed_whole(e, t)
        dec = feed_portions(e, t, [40, 1])
    close16(got, want)
    close16(dec, want)
    # a row whose streams nearly cancel in the final sum has its rounding blown up by the last norm: the others stay close
    size = np.linalg.norm(streams[-1], axis=-1)
    assert rel_err(got, want)[size > 0.5 * np.median(size)].max() < 0.3


def test_bfloat16_rows_with_clear_routing_stay_near_the_oracle(mix):
    cfg, W, d, o = mix
    t = toks(70, cfg["vocab"], 2)
    want = o.forward(t)
    clear = o.routing_margins(t) > 0.02
    assert clear.sum() >= 20
    with open_engine(d, dtype="bfloat16") as e:
        got = feed_whole(e, t)
        dec = feed_portions(e, t, [40, 1])
    for g in (got, dec):
        r = rel_err(g, want)
        assert np.median(r) < 0.06 and np.quantile(r[clear], 0.9) < 0.2


def test_bfloat16_widths_the_tensor_core_projection_cannot_take(tmp_path):
    """A width and inner sizes that are no multiple of 8 run on the general linear kernels."""
    layers = [parallel(l=left(dim=6, rot_dims=4), r=right(heads=3, dim=5, vdim=3, rot_dims=4), mlp=moe(ff=7)), mamba(inner=13, state=5, dt_rank=3)]
    cfg, W, d = build(tmp_path, layers, width=20, vocab=33)
    t = toks(40, 33, 4)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d, dtype="bfloat16") as e:
        close16(feed_whole(e, t), want)
    with open_engine(d) as e:
        close32(feed_whole(e, t), want)


def test_bfloat16_large_step_takes_the_per_expert_path_and_agrees_with_the_grouped_one(tmp_path, monkeypatch):
    """A step of several hundred tokens sorts rows per expert and runs every expert as one tensor-core product (identity
    experts keep their rows in the order and are skipped); the grouped tile kernel must give the same logits up to bf16
    rounding."""
    cfg, W, d = build(tmp_path, [parallel(l=left(chunk=40), mlp=moe(experts=4, identity=2, top=3, ff=16)), mamba(inner=32, state=8, mlp=moe(experts=3, identity=1, top=2, ff=16))],
                      seed=13, width=32)
    t = toks(300, cfg["vocab"], 14)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d, dtype="bfloat16") as e:
        big = feed_whole(e, t)
    monkeypatch.setenv("B200_NG_MOE_TC_MIN_T", "100000")
    with open_engine(d, dtype="bfloat16") as e:
        grouped = feed_whole(e, t)
    close16(big, want)
    close16(grouped, want)
    assert np.median(rel_err(big, grouped.astype(np.float64))) < 0.03


@pytest.mark.parametrize("heads,kv_heads,dim,chunk", [(4, 1, 16, 100), (2, 2, 32, 70), (6, 2, 64, 33), (8, 4, 128, 150), (3, 3, 16, 500), (12, 2, 48, 64), (8, 1, 16, 16)])
def test_bfloat16_tensor_core_attention_equals_the_general_kernel(tmp_path, monkeypatch, heads, kv_heads, dim, chunk):
    """Head sizes that fit the mma fragments take the tensor-core kernel in steps that bring prompt portions: several key
    tiles per chunk, chunk borders inside a tile of query rows, groups of 1 to 8 query heads per key head, portions that
    start in the middle of a tile, the sink in the finish.  The general kernel on the same bf16 cache must agree far inside
    bf16's distance to the oracle."""
    layers = [parallel(l=left(heads=heads, kv_heads=kv_heads, dim=dim, chunk=chunk, rot_dims=dim // 2, scale=2.0 / dim ** 0.5), mlp=None)]
    cfg, W, d = build(tmp_path, layers, seed=21, width=32)
    t = toks(230, cfg["vocab"], 22)
    want = oracle_for(cfg, W).forward(t)
    out = {}
    for knob in ("1", "0"):
        monkeypatch.setenv("B200_WATTN_MMA", knob)
        with open_engine(d, dtype="bfloat16") as e:
            out[knob] = (feed_whole(e, t), feed_portions(e, t, [70, 37, 64, 5, 1]))
    for a, b in zip(out["1"], out["0"]):
        close16(a, want)
        assert np.median(rel_err(a, b.astype(np.float64))) < 0.012 and rel_err(a, b.astype(np.float64)).max() < 0.05


def run_plan(e, seqs, plan):
    """Feed the sequences side by side: plan[step][i] tokens of sequence i per step (0: it sits the step out; past the plan's
    end every unfinished sequence brings one token).  Returns every sequence's logits."""
    rids = [e.feed_open() for _ in seqs]
    at, got, step = [0] * len(seqs), [[] for _ in seqs], 0
    while any(at[i] < len(seqs[i]) for i in range(len(seqs))):
        entries, idx = [], []
        for i in range(len(seqs)):
            n = min(plan[min(step, len(plan) - 1)][i] or (1 if step >= len(plan) else 0), len(seqs[i]) - at[i])
            if n > 0:
                entries.append((rids[i], seqs[i][at[i]:at[i] + n], list(range(n))))
                idx.append((i, n))
        out = e.feed_step(entries)
        r = 0
        for i, n in idx:
            got[i].append(out[r:r + n])
            at[i] += n
            r += n
        step += 1
    for r in rids:
        e.feed_close(r)
    return [np.concatenate(g) for g in got]


def test_bfloat16_mixed_batches_on_the_tensor_core_kernel_equal_each_request_alone(tmp_path, monkeypatch):
    layers = [parallel(l=left(heads=4, kv_heads=2, dim=32, chunk=40, rot_dims=16, scale=0.35), mlp=moe(experts=3, identity=0, top=3, ff=16)), mamba(inner=32, state=8, mlp=None)]
    cfg, W, d = build(tmp_path, layers, seed=71, width=32)
    o = oracle_for(cfg, W)
    seqs = [toks(n, cfg["vocab"], 72 + i) for i, n in enumerate((150, 61, 9, 120))]
    plan = [(70, 1, 9, 33), (37, 1, 0, 2), (1, 40, 0, 64), (42, 1, 0, 1), (0, 18, 0, 20)]
    monkeypatch.setenv("B200_WATTN_MMA", "1")
    with open_engine(d, dtype="bfloat16", max_tokens=160) as e:
        got = run_plan(e, seqs, plan)
        alone = [feed_whole(e, t) for t in seqs]
    for i in range(4):
        close16(got[i], o.forward(seqs[i]))
        assert np.median(rel_err(got[i], alone[i].astype(np.float64))) < 0.012 and rel_err(got[i], alone[i].astype(np.float64)).max() < 0.06


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_medium_sizes_on_every_projection_path(tmp_path, dtype):
    layers = [parallel(l=left(heads=4, kv_heads=2, dim=16, chunk=33), r=right(heads=2, dim=16, vdim=24), mlp=moe(experts=6, identity=2, top=3, ff=40)),
              mamba(inner=144, state=16, dt_rank=5, mlp=moe(experts=6, identity=2, top=3, ff=40))]
    cfg, W, d = build(tmp_path, layers, seed=17, width=72, vocab=90)
    t = toks(150, 90, 18)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d, dtype=dtype) as e:
        whole = feed_whole(e, t)
        parts = feed_portions(e, t, [70, 9, 1])
    (close32 if dtype == "float32" else close16)(whole, want)
    (close32 if dtype == "float32" else close16)(parts, want)


# ---------------------------------------------------------------- cutting a sequence
def test_prefill_equals_token_by_token_decoding(mix):
    cfg, W, d, o = mix
    t = toks(45, cfg["vocab"], 3)
    with open_engine(d) as e:
        whole = feed_whole(e, t)
        single = feed_portions(e, t, [1])
    close32(whole, o.forward(t))
    assert np.abs(whole - single).max() < 2e-4 * np.abs(whole).max()


@pytest.mark.parametrize("sizes", [[2], [3, 2], [16, 1], [17, 5, 2], [5, 16, 16, 2, 1], [1, 1, 2, 1, 3]])
def test_portions_of_any_size_give_the_same_logits(mix, sizes):
    cfg, W, d, o = mix
    t = toks(61, cfg["vocab"], 5)
    with open_engine(d) as e:
        got = feed_portions(e, t, sizes)
    close32(got, o.forward(t))


@pytest.mark.parametrize("taps", [2, 4, 7])
def test_carried_convolution_inputs_survive_portions_shorter_than_the_taps(tmp_path, taps):
    """Portions of one and two tokens under a convolution of up to seven taps: the slot's carried inputs are shifted, not
    replaced, and a later portion still reads inputs of three steps ago."""
    cfg, W, d = build(tmp_path, [parallel(l=left(conv=taps), mlp=None), mamba(conv=taps, mlp=None)], seed=6)
    t = toks(33, cfg["vocab"], 7)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d) as e:
        close32(feed_portions(e, t, [1, 2, 1, 1, 2, 5, 1, 2, 2, 1]), want)
        close32(feed_portions(e, t, [taps - 1, taps, 1, taps + 1, 2]), want)


def test_long_decoding_stays_on_the_oracle(tmp_path):
    cfg, W, d = build(tmp_path, [parallel(l=left(chunk=20)), mamba(mlp=None), parallel(r=right(decay=[0.97, 0.999]), mlp=None)], seed=8)
    t = toks(260, cfg["vocab"], 7)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d) as e:
        got = feed_portions(e, t, [20, 1])
    close32(got, want, 5)


# ---------------------------------------------------------------- batches, pages, slots
def test_unequal_requests_in_one_batch_equal_each_alone(mix):
    cfg, W, d, o = mix
    seqs = [toks(n, cfg["vocab"], 10 + i) for i, n in enumerate((50, 23, 9, 77))]
    plan = [(7, 1, 9, 30), (20, 1, 0, 2), (1, 3, 0, 17), (22, 1, 0, 1), (0, 17, 0, 27)]
    with open_engine(d, max_tokens=128) as e:
        got = run_plan(e, seqs, plan)
    for i in range(4):
        close32(got[i], o.forward(seqs[i]))


def feed_portions_on(e, r, tokens, sizes):
    outs, at, i = [], 0, 0
    while at < len(tokens):
        n = min(sizes[min(i, len(sizes) - 1)], len(tokens) - at)
        outs.append(e.feed_step([(r, tokens[at:at + n], list(range(n)))]))
        at += n
        i += 1
    e.feed_close(r)
    return np.concatenate(outs)


def test_pages_and_slots_are_used_again(mix_wide):
    """A pool of exactly two sequences' pages and two slots: later requests run in what earlier ones gave back, and start
    from empty states and empty carried inputs whatever the slot held."""
    cfg, W, d, o = mix_wide
    seqs = [toks(n, cfg["vocab"], 20 + i) for i, n in enumerate((40, 33, 48, 17, 41))]
    with open_engine(d, max_tokens=48, max_seqs=2, blocks=6, budget=96) as e:
        a, b = e.feed_open(), e.feed_open()
        e.feed_step([(a, seqs[0], []), (b, seqs[1][:20], [])])
        e.feed_step([(b, seqs[1][20:], [])])
        e.feed_close(a)
        c = e.feed_open()                      # takes a's slot and pages while b is still live
        got_c = e.feed_step([(c, seqs[2][:30], list(range(30)))])
        e.feed_close(b)
        f = e.feed_open()
        out = e.feed_step([(c, seqs[2][30:], list(range(18))), (f, seqs[3], list(range(17)))])
        got_c = np.concatenate([got_c, out[:18]])
        got_f = out[18:]
        e.feed_close(c)
        e.feed_close(f)
        g = e.feed_open()
        got_g = feed_portions_on(e, g, seqs[4], [16, 1])
        assert e.stats().kv_blocks_free == 6
    close32(got_c, o.forward(seqs[2]))
    close32(got_f, o.forward(seqs[3]))
    close32(got_g, o.forward(seqs[4]))


def test_pages_behind_every_chunk_go_back_while_the_sequences_run(tmp_path):
    """Two 380-token sequences side by side in a pool that could not hold both whole: a token never looks behind the start
    of its chunk, so the pages before every layer's chunk are returned while the sequences run."""
    cfg, W, d = build(tmp_path, [parallel(l=left(chunk=20)), mamba(mlp=None), parallel(l=left(chunk=33), mlp=None)], seed=61)
    o = oracle_for(cfg, W)
    seqs = [toks(380, cfg["vocab"], 62 + i) for i in range(2)]
    want = [o.forward(t) for t in seqs]
    with open_engine(d, max_tokens=400, max_seqs=2, blocks=30, budget=64) as e:
        rids = [e.feed_open() for _ in seqs]
        got = [[], []]
        at = 0
        sizes = [16, 7, 16, 1, 2, 16]
        i = 0
        while at < 380:
            n = min(sizes[i % len(sizes)], 380 - at)
            out = e.feed_step([(r, t[at:at + n], list(range(n))) for r, t in zip(rids, seqs)])
            got[0].append(out[:n])
            got[1].append(out[n:])
            at += n
            i += 1
            assert e.stats().kv_blocks_free >= 30 - 2 * 5       # chunk 33 + a 16-token portion: at most 5 pages each
        for r in rids:
            e.feed_close(r)
        assert e.stats().kv_blocks_free == 30
    for k in range(2):
        close32(np.concatenate(got[k]), want[k], 3)


def test_a_step_over_the_pool_is_refused_and_leaves_the_engine_usable(mix_wide):
    from kubeai_b200 import B200Error
    cfg, W, d, o = mix_wide
    t = toks(40, cfg["vocab"], 30)
    with open_engine(d, max_tokens=48, max_seqs=2, blocks=3) as e:
        a, b = e.feed_open(), e.feed_open()
        e.feed_step([(a, t[:30], [])])
        with pytest.raises(B200Error):
            e.feed_step([(b, t[:30], [])])        # 2 + 2 pages do not fit 3
        got = e.feed_step([(a, t[30:], list(range(10)))])
        e.feed_close(a)
        e.feed_close(b)
    close32(got, o.forward(t)[30:])


def test_a_sequence_cannot_outgrow_the_position_table(tmp_path):
    from kubeai_b200 import B200Error
    cfg, W, d = build(tmp_path, [mamba(mlp=None)], max_positions=40)
    t = toks(41, cfg["vocab"], 1)
    with open_engine(d, max_tokens=128) as e:
        close32(feed_whole(e, t[:40]), oracle_for(cfg, W).forward(t[:40]))
        r = e.feed_open()
        with pytest.raises(B200Error):
            e.feed_step([(r, t, [])])
        e.feed_close(r)


# ---------------------------------------------------------------- edges made visible
QTOK, KTOK = 7, 11


def edge_model(tmp_path, chunk, seed=31):
    """One layer whose left branch copies from KTOK positions whenever a QTOK position can see one (planted pair, sharp
    softmax, no rotation, no convolution, no position rows); the right branch is switched off so that nothing else carries
    KTOK forward."""
    cfg = make_config([parallel(l=left(heads=2, kv_heads=1, dim=16, chunk=chunk, rot_dims=0, scale=6.0, conv=0), mlp=None)], width=48, vocab=40, max_positions=512)
    W = plant_pair(cfg, random_weights(cfg, seed=seed, pos_gain=0.0, left_only=True), QTOK, KTOK)
    return cfg, W, write_model_dir(tmp_path / ("m%d" % chunk), cfg, W)


def sequence_with(n, key_at, query_at, seed):
    """Random filler without the two special tokens, KTOK at key_at, QTOK at query_at."""
    t = [x for x in np.random.default_rng(seed).integers(12, 40, size=n).tolist()]
    t[key_at] = KTOK
    t[query_at] = QTOK
    return t


@pytest.mark.parametrize("chunk,nchunk,qoff", [(17, 2, 16), (16, 2, 15), (16, 3, 1), (64, 1, 63), (5, 6, 4), (48, 4, 47), (33, 3, 1), (2, 20, 1)])
def test_chunk_edge_is_exact_in_prompts_and_in_decoding(tmp_path, chunk, nchunk, qoff):
    """The key on the first position of the query's chunk decides the query's logits, the key one position earlier (the last
    of the chunk before) is invisible: the oracle's own logits differ strongly between the two placements, and the engine
    follows it in both, in a prompt step, in portions that cut between key and query or at the chunk's border, and token by
    token.  The query sits on the chunk's last position (the far edge) or on its second."""
    cfg, W, d = edge_model(tmp_path, chunk)
    o = oracle_for(cfg, W)
    start = nchunk * chunk
    qpos = start + qoff
    inside = sequence_with(qpos + 3, start, qpos, 1)
    outside = sequence_with(qpos + 3, start - 1, qpos, 1)
    w_in, w_out = o.forward(inside), o.forward(outside)
    assert rel_err(w_in[qpos:qpos + 1], w_out[qpos:qpos + 1])[0] > 0.3      # the placement matters
    with open_engine(d) as e:
        for t, want in ((inside, w_in), (outside, w_out)):
            close32(feed_whole(e, t), want)
            close32(feed_portions(e, t, [qpos - 1, 2, 1] if qpos > 2 else [1]), want)
            close32(feed_portions(e, t, [start, 1] if qoff < 3 else [start, qoff - 1, 1]), want)
            close32(feed_portions(e, t, [start - 1, 2, 1]), want)
    with open_engine(d, dtype="bfloat16") as e:
        for t, want in ((inside, w_in), (outside, w_out)):
            assert np.median(rel_err(feed_whole(e, t), want)) < 0.1
            assert rel_err(feed_portions(e, t, [qpos, 1]), want)[qpos] < 0.25


def test_the_first_position_of_a_chunk_sees_itself_alone(tmp_path):
    """A query on a chunk's first position has one key, its own: whatever stands before changes nothing in its logits."""
    cfg, W, d = edge_model(tmp_path, 16)
    o = oracle_for(cfg, W)
    a = sequence_with(40, 31, 32, 4)
    b = sequence_with(40, 5, 32, 9)
    wa, wb = o.forward(a), o.forward(b)
    assert np.abs(wa[32] - wb[32]).max() < 1e-9
    with open_engine(d) as e:
        ga, gb = feed_whole(e, a), feed_portions(e, b, [32, 1])
    assert np.abs(ga[32] - gb[32]).max() < 1e-4 * np.abs(ga[32]).max()
    close32(ga, wa)


def test_a_far_key_inside_a_long_chunk_is_found_among_hundreds(tmp_path):
    cfg, W, d = edge_model(tmp_path, 400)
    o = oracle_for(cfg, W)
    near = sequence_with(420, 3, 395, 3)             # 392 back, same chunk, 24 pages away
    gone = sequence_with(420, 399, 410, 3)           # 11 back, but in the chunk before
    w_near, w_gone = o.forward(near), o.forward(gone)
    without = list(near)
    without[3] = 13
    assert rel_err(w_near[395:396], o.forward(without)[395:396])[0] > 0.3      # the far key decides
    without = list(gone)
    without[399] = 13
    assert rel_err(w_gone[410:411], o.forward(without)[410:411])[0] < 1e-9     # the near key of the other chunk does not count
    with open_engine(d) as e:
        close32(feed_whole(e, near), w_near)
        close32(feed_portions(e, gone, [405, 1]), w_gone)
        close32(feed_portions(e, near, [100, 33, 2]), w_near)
        close32(feed_portions(e, near, [390, 1]), w_near)
    with open_engine(d, dtype="bfloat16") as e:
        assert rel_err(feed_whole(e, near), w_near)[395] < 0.25
        assert rel_err(feed_portions(e, near, [390, 1]), w_near)[395] < 0.25


def test_the_sink_takes_its_share_of_the_softmax(tmp_path):
    """A large sink empties the attention, a very negative one leaves the plain softmax: both follow the oracle, and differ."""
    cfg = make_config([parallel(l=left(heads=2, kv_heads=1, dim=8, chunk=12, scale=0.5), mlp=None)], width=24)
    W = random_weights(cfg, seed=15, left_only=True)
    t = toks(30, cfg["vocab"], 16)
    outs = []
    for i, sink in enumerate((6.0, -30.0)):
        Ws = dict(W)
        Ws["l0.mix.left.sink"] = np.full(2, sink, dtype=np.float32)
        d = write_model_dir(tmp_path / ("s%d" % i), cfg, Ws)
        want = oracle_for(cfg, Ws).forward(t)
        with open_engine(d) as e:
            close32(feed_whole(e, t), want)
            close32(feed_portions(e, t, [13, 1]), want)
        with open_engine(d, dtype="bfloat16") as e:
            close16(feed_whole(e, t), want)
        outs.append(want)
    assert rel_err(outs[0], outs[1]).max() > 0.1


def test_far_tokens_reach_through_the_retention_state(tmp_path):
    """With a decay close to one the right branch carries a token across hundreds of positions: changing the first token
    changes the last logits, and the engine follows the oracle whether the prompt comes whole, in portions or decoded."""
    cfg, W, d = build(tmp_path, [parallel(l=left(chunk=4), r=right(heads=2, dim=8, vdim=8, decay=[0.9999, 0.9995]), mlp=None)], seed=41, wkw=RIGHT)
    o = oracle_for(cfg, W)
    a = toks(300, cfg["vocab"], 42)
    b = [(a[0] + 1) % cfg["vocab"]] + a[1:]
    wa, wb = o.forward(a), o.forward(b)
    assert rel_err(wa[-1:], wb[-1:])[0] > 0.01
    with open_engine(d) as e:
        close32(feed_whole(e, a), wa, 3)
        close32(feed_portions(e, b, [150, 33, 1]), wb, 3)


def test_far_tokens_reach_through_the_scan_state(tmp_path):
    """Slow channels (A close to zero) keep the first tokens in the scan state for hundreds of positions."""
    cfg = make_config([mamba(inner=24, state=8, dt_rank=3, mlp=None)])
    W = random_weights(cfg, seed=43)
    W["l0.mix.A_log"][:] = np.float32(-8.0)
    d = write_model_dir(tmp_path / "m", cfg, W)
    o = oracle_for(cfg, W)
    a = toks(300, cfg["vocab"], 44)
    b = [(x + 1) % cfg["vocab"] for x in a[:30]] + a[30:]        # other first tokens, the same last 270
    wa, wb = o.forward(a), o.forward(b)
    assert rel_err(wa[-1:], wb[-1:])[0] > 0.01
    with open_engine(d) as e:
        close32(feed_whole(e, a), wa, 3)
        close32(feed_portions(e, b, [150, 33, 1]), wb, 3)


def test_first_tokens_of_a_sequence(mix):
    cfg, W, d, o = mix
    with open_engine(d) as e:
        for n in (1, 2, 3):
            t = toks(n, cfg["vocab"], 50 + n)
            close32(feed_whole(e, t), o.forward(t))
        t = toks(6, cfg["vocab"], 54)
        close32(feed_portions(e, t, [1, 1, 2]), o.forward(t))


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(tmp_path, seed):
    rng = np.random.default_rng(100 + seed)
    layers = []

    def rand_moe():
        if rng.random() < 0.3:
            return None
        E, I = int(rng.integers(1, 8)), int(rng.integers(0, 4))
        return moe(experts=E, identity=I, top=int(rng.integers(1, E + I + 1)), ff=int(rng.integers(1, 20)), limit=float(rng.uniform(0.3, 3.0)))

    for _ in range(int(rng.integers(1, 5))):
        if rng.random() < 0.5:
            G = int(rng.integers(1, 4))
            D = int(rng.integers(2, 13))
            l = left(heads=G * int(rng.integers(1, 4)), kv_heads=G, dim=D, chunk=int(rng.integers(0, 40)), rot_dims=2 * int(rng.integers(0, D // 2 + 1)),
                     scale=float(rng.uniform(0.1, 0.6)), conv=int(rng.integers(0, 6)))
            Hr, Dr = int(rng.integers(1, 4)), int(rng.integers(1, 20))
            r = right(heads=Hr, dim=Dr, vdim=int(rng.integers(1, 20)), decay=[float(x) for x in rng.uniform(0.3, 0.999, size=Hr)],
                      rot_dims=2 * int(rng.integers(0, Dr // 2 + 1)))
            layers.append(parallel(l=l, r=r, mlp=rand_moe()))
        else:
            layers.append(mamba(inner=int(rng.integers(1, 40)), state=int(rng.integers(1, 24)), dt_rank=int(rng.integers(1, 6)), conv=int(rng.integers(1, 6)),
                                mlp=rand_moe()))
    streams = [None, 1, 2, 4][int(rng.integers(0, 4))]
    cfg, W, d = build(tmp_path, layers, seed=200 + seed, width=int(rng.integers(6, 40)), vocab=int(rng.integers(5, 60)), streams=streams,
                      logit_scale=float(rng.uniform(0.3, 2.0)), wkw=dict(gated=bool(rng.random() < 0.8)))
    t = toks(70, cfg["vocab"], seed)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d) as e:
        close32(feed_whole(e, t), want, 3)
        close32(feed_portions(e, t, [int(rng.integers(2, 30)), int(rng.integers(1, 9)), 1]), want, 3)


@pytest.mark.parametrize("seed", range(4))
def test_bfloat16_random_medium_configurations(tmp_path, seed):
    """Sizes that the tensor-core projections, the tensor-core attention and the per-expert path take (widths and head sizes
    in multiples of 16, a step of 300 tokens), in random layer orders: the bf16 engine stays near the oracle on rows whose
    routing is clear, whole and in portions, and the fp32 engine on all rows."""
    rng = np.random.default_rng(300 + seed)
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    Wd = pick([64, 96, 128, 192])
    layers = []
    for _ in range(int(rng.integers(2, 5))):
        E, I = pick([3, 4, 8]), pick([0, 1, 2])
        mlp = None if rng.random() < 0.2 else moe(experts=E, identity=I, top=pick([1, 2, 3]), ff=pick([32, 48, 96]), limit=float(rng.uniform(1.0, 4.0)))
        if rng.random() < 0.55:
            G = pick([1, 2])
            D = pick([16, 32, 48, 64])
            Dr = pick([16, 32])
            layers.append(parallel(l=left(heads=G * pick([1, 2, 4]), kv_heads=G, dim=D, chunk=pick([24, 32, 64, 100]), rot_dims=pick([D, D // 2]), scale=D ** -0.5, conv=pick([2, 3, 4]),
                                          base=pick([100.0, 50000.0])),
                                   r=right(heads=pick([2, 4]), dim=Dr, vdim=pick([16, 32, 64]), rot_dims=pick([Dr, Dr // 2]), base=1e6), mlp=mlp))
            layers[-1]["mixer"]["right"]["decay"] = [float(1.0 - 2.0 ** -rng.uniform(3, 10)) for _ in range(layers[-1]["mixer"]["right"]["heads"])]
        else:
            layers.append(mamba(inner=pick([Wd, 2 * Wd]), state=pick([8, 16, 32]), dt_rank=max(1, Wd // 16), conv=pick([2, 4]), mlp=mlp))
    cfg, W, d = build(tmp_path, layers, seed=400 + seed, width=Wd, vocab=pick([64, 250]), streams=pick([1, 2, 3, 4]), logit_scale=float(rng.uniform(0.4, 1.5)))
    o = oracle_for(cfg, W)
    t = toks(300, cfg["vocab"], seed)
    want = o.forward(t)
    clear = o.routing_margins(t) > 0.02
    with open_engine(d) as e:
        close32(feed_whole(e, t), want, 3)
    with open_engine(d, dtype="bfloat16") as e:
        whole = feed_whole(e, t)
        parts = feed_portions(e, t, [130, 70, 33, 2, 1])
    for g in (whole, parts):
        r = rel_err(g, want)
        assert np.median(r) < 0.06 and np.quantile(r[clear], 0.9) < 0.2, (np.median(r), np.quantile(r[clear], 0.9))


# ---------------------------------------------------------------- the engine's own generation path
def greedy_agrees(o, prompt, got):
    want, margin = o.generate(prompt, len(got))
    if margin > 1e-3:
        assert got == want
    else:      # a tie within fp32 rounding may go either way: agree up to the first close call
        k = 0
        while k < len(got) and got[k] == want[k]:
            k += 1
        assert k >= 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_submit_scheduler_and_sampler(mix, dtype):
    """More requests than slots, a token budget that cuts prompts into portions, generation by the engine's argmax."""
    cfg, W, d, o = mix
    prompts = [toks(n, cfg["vocab"], 40 + i) for i, n in enumerate((37, 5, 21, 50, 2))]
    with open_engine(d, dtype=dtype, max_tokens=96, max_seqs=2, budget=16, blocks=12) as e:
        outs = e.generate(prompts, max_tokens=12)
        st = e.stats()
    assert st.kv_blocks_free == 12
    for p, got in zip(prompts, outs):
        assert len(got) == 12
        if dtype == "float32":
            greedy_agrees(o, p, got)
    if dtype == "bfloat16":
        for p, got in zip(prompts, outs):
            row = np.sort(o.forward(p)[-1])
            if row[-1] - row[-2] > 0.3:
                assert got[0] == int(np.argmax(o.forward(p)[-1]))


def test_preemption_recomputes_cache_and_state_from_the_start(mix_wide):
    """A pool too small for all running sequences to finish: the scheduler preempts and recomputes; outputs do not change."""
    cfg, W, d, o = mix_wide
    prompts = [toks(n, cfg["vocab"], 60 + i) for i, n in enumerate((30, 28, 31))]
    with open_engine(d, max_tokens=64, max_seqs=3, budget=64, blocks=8) as e:
        outs = e.generate(prompts, max_tokens=20)
        assert e.stats().preemptions > 0
    for p, got in zip(prompts, outs):
        greedy_agrees(o, p, got)


def test_chat_completion_through_the_serving_shell(tmp_path):
    """The design behind the HTTP handler chain, stepped by the engine's own background loop: prompt rendering, submit,
    continuous batching of two concurrent requests, greedy sampling, SSE framing; the tokens are the oracle's."""
    import json
    import threading
    from kubeai_b200.engine import Engine, default_config
    from kubeai_b200.server import Server, tokenize
    V = 300
    cfg, W, d = build(tmp_path, MIX, seed=51, vocab=V, max_positions=256)
    o = oracle_for(cfg, W)
    lim = default_config(manual_step=0, enable_prefix_caching=0, max_num_seqs=4, max_batched_tokens=32, max_model_len=256, num_kv_blocks=64)
    eng = Engine(lim, d, dtype="float32")
    srv = Server([eng], model="nx", vocab=V, max_model_len=256)
    try:
        out = {}

        def ask(i, text):
            body = dict(model="nx", messages=[{"role": "user", "content": text}], max_tokens=5, temperature=0, stream=(i == 0))
            out[i] = srv.handle("POST", "/openai/v1/chat/completions", json.dumps(body))

        th = [threading.Thread(target=ask, args=(i, t)) for i, t in enumerate(["Hello there, how are you?", "Hi"])]
        for t in th:
            t.start()
        for t in th:
            t.join()
        assert out[0].status == 200 and out[1].status == 200
        ev = out[0].sse_events()
        assert ev[-1] == "[DONE]"
        text0 = "".join(json.loads(e)["choices"][0]["delta"].get("content", "") for e in ev[:-1] if json.loads(e)["choices"])
        text1 = out[1].json()["choices"][0]["message"]["content"]
        for text, user in ((text0, "Hello there, how are you?"), (text1, "Hi")):
            prompt = srv.render_prompt("/v1/chat/completions", json.dumps(dict(model="nx", messages=[{"role": "user", "content": user}])))
            got = tokenize(text, V)
            assert len(got) == 5
            greedy_agrees(o, prompt, got)
    finally:
        srv.close()
        eng.close()


def test_a_checkpoint_without_a_tensor_the_config_asks_for_is_refused(tmp_path):
    from kubeai_b200 import B200Error
    from kubeai_b200.engine import Engine, default_config
    cfg = make_config([parallel(), mamba()])
    for i, name in enumerate(["l0.hc2.mix", "l0.mix.left.sink", "l1.mix.A_log", "pos", "l1.rg2.b"]):
        short = random_weights(cfg)
        del short[name]
        with pytest.raises(B200Error, match=name):
            Engine(default_config(manual_step=1), write_model_dir(tmp_path / ("c%d" % i), cfg, short), dtype="float32")
