"""Mulenex through the engine against the plain oracle (oracle/mulenex_oracle.py): each mechanism alone, prefill against
token-by-token decoding, portions down to two tokens, unequal batches, pages and slots used again, far keys and keys at
page borders made visible by a planted query/key pair, the causal edge, the steps of the query gain, the first tokens of
the recurrence, other sizes (also the degenerate ones), long decoding, and greedy generation through the engine's own
submit / scheduler / sampling path.  Configurations and weights are made here; nothing is read from disk but what the
test wrote."""
import numpy as np
import pytest

from mulenex_util import (attention, dense, feed_portions, feed_whole, layer, make_config, mlstm, moe, open_engine, oracle_for, plant_pair,
                          random_weights, rel_err, write_model_dir)

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


def build(tmp_path, layers, seed=0, width=24, vocab=40, eps=1e-5, **kw):
    cfg = make_config(layers, width=width, vocab=vocab, eps=eps)
    W = random_weights(cfg, seed=seed, **kw)
    return cfg, W, write_model_dir(tmp_path / "m", cfg, W)


# a recurrent layer first, attention layers of different shapes, blending that starts in the middle, every kind of feed-forward
MIX = [layer(mlstm(), mlp=dense()),
       layer(attention(heads=3, kv_heads=3, dim=6, vdim=4, v_mix=False, softcap=None), mlp=None),
       layer(attention()),
       layer(mlstm(heads=3, dim=4, vdim=6, gate_cap=4.0), mlp=moe(experts=7, top=1, shared=None)),
       layer(attention(heads=2, kv_heads=2, dim=10, q_temp=None), mlp=dense(ff=9))]


@pytest.fixture(scope="module")
def mix(tmp_path_factory):
    cfg, W, d = build(tmp_path_factory.mktemp("mix"), MIX)
    return cfg, W, d, oracle_for(cfg, W)


# ---------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("name,layers,kw", [
    ("attention_only", [layer(attention(v_mix=False), mlp=None)], {}),
    ("attention_full_heads_no_cap_no_gain", [layer(attention(heads=3, kv_heads=3, softcap=None, q_temp=None, v_mix=False), mlp=None)], {}),
    ("attention_one_kv_head", [layer(attention(heads=4, kv_heads=1, dim=4, vdim=9), mlp=None)], {}),
    ("attention_tight_cap", [layer(attention(scale=3.0, softcap=0.8), mlp=None)], {}),
    ("attention_gain_every_position", [layer(attention(q_temp=(1.5, 1)), mlp=None)], {}),
    ("attention_odd_head_size", [layer(attention(dim=7, vdim=5), mlp=None)], {}),
    ("blend_from_the_second_attention", [layer(attention(v_mix=False), mlp=None), layer(attention(), mlp=None), layer(attention(), mlp=None),
                                         layer(attention(v_mix=False), mlp=None), layer(attention(heads=2, kv_heads=2, dim=10), mlp=None)], {}),
    ("blend_everything", [layer(attention(), mlp=None), layer(attention(), mlp=None)], dict(lam=1.0)),
    ("mlstm_only", [layer(mlstm(), mlp=None)], {}),
    ("mlstm_one_head_wide_value", [layer(mlstm(heads=1, dim=4, vdim=40), mlp=None)], {}),
    ("mlstm_many_rows", [layer(mlstm(heads=2, dim=40, vdim=8), mlp=None)], {}),
    ("mlstm_strong_input_gate", [layer(mlstm(gate_cap=12.0), mlp=None)], dict(gate_bias=(6.0, 3.0))),
    ("mlstm_weak_input_gate", [layer(mlstm(gate_cap=12.0), mlp=None)], dict(gate_bias=(-7.0, 4.0))),
    ("mlstm_forgetful", [layer(mlstm(gate_cap=12.0), mlp=None)], dict(gate_bias=(1.0, -6.0))),
    ("mlstm_tight_gate_cap", [layer(mlstm(gate_cap=0.5), mlp=None)], dict(gate_bias=(2.0, 2.0))),
    ("dense", [layer(mlp=dense())], {}),
    ("moe_with_shared", [layer()], {}),
    ("moe_top1_no_shared", [layer(mlp=moe(top=1, shared=None))], {}),
    ("moe_all_experts", [layer(mlp=moe(experts=3, top=3))], {}),
    ("moe_one_expert", [layer(mlp=moe(experts=1, top=1, shared=5))], {}),
    ("odd_width", [layer(), layer(mlstm())], dict(width=21, vocab=33)),
    ("large_eps_in_every_norm", [layer(), layer(mlstm(), mlp=dense())], dict(eps=0.05)),
])
def test_each_mechanism_matches_the_oracle(tmp_path, name, layers, kw):
    cfg, W, d = build(tmp_path, layers, seed=3, **kw)
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
    """Without routing decisions (every expert chosen) bf16 rounding moves every row by a few percent at most."""
    layers = [layer(mlp=moe(experts=3, top=3)), MIX[0], MIX[1], layer(attention(heads=2, kv_heads=2), mlp=moe(experts=2, top=2, shared=None))]
    cfg, W, d = build(tmp_path, layers, seed=9)
    t = toks(70, cfg["vocab"], 2)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d, dtype="bfloat16") as e:
        got = feed_whole(e, t)
        dec = feed_portions(e, t, [40, 1])
    close16(got, want)
    close16(dec, want)
    assert rel_err(got, want).max() < 0.3


def test_bfloat16_rows_with_clear_routing_stay_near_the_oracle(mix):
    cfg, W, d, o = mix
    t = toks(70, cfg["vocab"], 2)
    want = o.forward(t)
    clear = o.routing_margins(t) > 0.05
    assert clear.sum() >= 20
    with open_engine(d, dtype="bfloat16") as e:
        got = feed_whole(e, t)
        dec = feed_portions(e, t, [40, 1])
    for g in (got, dec):
        r = rel_err(g, want)
        assert np.median(r) < 0.06 and np.quantile(r[clear], 0.9) < 0.2


def test_bfloat16_widths_the_tensor_core_projection_cannot_take(tmp_path):
    """A width and inner sizes that are no multiple of 8 run on the general linear kernels."""
    layers = [layer(attention(dim=6, vdim=5), mlp=moe(ff=7, shared=9)), layer(mlstm(heads=3, dim=5, vdim=3), mlp=dense(ff=11))]
    cfg, W, d = build(tmp_path, layers, width=20, vocab=33)
    t = toks(40, 33, 4)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d, dtype="bfloat16") as e:
        close16(feed_whole(e, t), want)
    with open_engine(d) as e:
        close32(feed_whole(e, t), want)


def test_bfloat16_tensor_core_projections_agree_with_the_general_ones(tmp_path, monkeypatch):
    layers = [layer(attention(heads=4, kv_heads=2, dim=16, vdim=8), mlp=dense(ff=48)), layer(mlstm(heads=2, dim=8, vdim=16), mlp=moe(experts=3, top=3, ff=16, shared=24))]
    cfg, W, d = build(tmp_path, layers, seed=12, width=32)
    t = toks(150, cfg["vocab"], 13)
    want = oracle_for(cfg, W).forward(t)
    out = {}
    for knob in ("1", "0"):
        monkeypatch.setenv("B200_MX_TC", knob)
        with open_engine(d, dtype="bfloat16") as e:
            out[knob] = feed_whole(e, t)
        close16(out[knob], want)
    assert np.median(rel_err(out["1"], out["0"].astype(np.float64))) < 0.03


def test_bfloat16_large_step_takes_the_per_expert_path_and_agrees_with_the_grouped_one(tmp_path, monkeypatch):
    """A step of several hundred tokens sorts rows per expert and runs every expert as one tensor-core product; the
    grouped tile kernel must give the same logits up to bf16 rounding."""
    cfg, W, d = build(tmp_path, [layer(mlp=moe(experts=4, top=2, ff=16, shared=16))], seed=13, width=32)
    t = toks(300, cfg["vocab"], 14)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d, dtype="bfloat16") as e:
        big = feed_whole(e, t)
    monkeypatch.setenv("B200_MX_MOE_TC_MIN_T", "100000")
    with open_engine(d, dtype="bfloat16") as e:
        grouped = feed_whole(e, t)
    close16(big, want)
    close16(grouped, want)
    assert np.median(rel_err(big, grouped.astype(np.float64))) < 0.03


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,cap", [(4, 1, 16, 16, 5.0), (2, 2, 32, 48, None), (6, 2, 64, 32, 20.0), (8, 4, 128, 128, 30.0), (3, 3, 16, 32, 1.5),
                                                           (4, 2, 48, 80, 10.0), (2, 1, 96, 112, None)])
def test_bfloat16_tensor_core_attention_equals_the_general_kernel(tmp_path, monkeypatch, heads, kv_heads, dim, vdim, cap):
    """Head sizes that fit the mma fragments take the tensor-core kernel in steps that bring prompt portions: several key
    tiles per sequence, groups of 1 to 4 query heads per key head, capped and uncapped scores, one gate per head, portions
    that start in the middle of a tile.  The general kernel on the same bf16 cache must agree far inside bf16's distance to
    the oracle."""
    layers = [layer(attention(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=2.0 / dim ** 0.5, softcap=cap, q_temp=(0.6, 50)), mlp=None)]
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_medium_sizes_on_every_projection_path(tmp_path, dtype):
    layers = [layer(attention(heads=4, kv_heads=2, dim=16, vdim=24), mlp=moe(experts=6, top=2, ff=40, shared=24)),
              layer(mlstm(heads=2, dim=16, vdim=24), mlp=dense(ff=100)), layer(attention(heads=4, kv_heads=2, dim=32, vdim=24), mlp=moe(experts=4, top=4, ff=24))]
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


@pytest.mark.parametrize("sizes", [[2], [3, 2], [16, 1], [17, 5, 2], [5, 16, 16, 2, 1]])
def test_portions_of_any_size_give_the_same_logits(mix, sizes):
    cfg, W, d, o = mix
    t = toks(61, cfg["vocab"], 5)
    with open_engine(d) as e:
        got = feed_portions(e, t, sizes)
    close32(got, o.forward(t))


def test_long_decoding_stays_on_the_oracle(tmp_path):
    cfg, W, d = build(tmp_path, [layer(attention(q_temp=(0.5, 64))), layer(mlstm(gate_cap=10.0), mlp=None)], seed=8, gate_bias=(0.5, 5.0))
    t = toks(260, cfg["vocab"], 7)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d) as e:
        got = feed_portions(e, t, [20, 1])
    close32(got, want, 5)


# ---------------------------------------------------------------- batches, pages, slots
def run_plan(e, seqs, plan):
    """Feed the sequences side by side, sequence i bringing plan[step][i] tokens (then one per step); logits of every position."""
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


def test_unequal_requests_in_one_batch_equal_each_alone(mix):
    cfg, W, d, o = mix
    seqs = [toks(n, cfg["vocab"], 10 + i) for i, n in enumerate((50, 23, 9, 77))]
    with open_engine(d, max_tokens=128) as e:
        got = run_plan(e, seqs, [(7, 1, 9, 30), (20, 1, 0, 2), (1, 3, 0, 17), (22, 1, 0, 1), (0, 17, 0, 27)])
    for g, t in zip(got, seqs):
        close32(g, o.forward(t))


def test_bfloat16_mixed_batches_on_the_tensor_core_kernel_equal_each_request_alone(tmp_path, monkeypatch):
    layers = [layer(attention(heads=4, kv_heads=2, dim=32, vdim=16, scale=0.35), mlp=moe(experts=3, top=3, ff=16, shared=16)), layer(mlstm(heads=2, dim=16, vdim=16), mlp=None),
              layer(attention(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.35), mlp=dense(ff=32))]
    cfg, W, d = build(tmp_path, layers, seed=71, width=32)
    o = oracle_for(cfg, W)
    seqs = [toks(n, cfg["vocab"], 72 + i) for i, n in enumerate((150, 61, 9, 120))]
    monkeypatch.setenv("B200_WATTN_MMA", "1")
    with open_engine(d, dtype="bfloat16", max_tokens=160) as e:
        got = run_plan(e, seqs, [(70, 1, 9, 33), (37, 1, 0, 2), (1, 40, 0, 64), (42, 1, 0, 1), (0, 18, 0, 20)])
        alone = [feed_whole(e, t) for t in seqs]
    for g, a, t in zip(got, alone, seqs):
        close16(g, o.forward(t))
        assert np.median(rel_err(g, a.astype(np.float64))) < 0.012 and rel_err(g, a.astype(np.float64)).max() < 0.06


def feed_portions_on(e, r, tokens, sizes):
    outs, at, i = [], 0, 0
    while at < len(tokens):
        n = min(sizes[min(i, len(sizes) - 1)], len(tokens) - at)
        outs.append(e.feed_step([(r, tokens[at:at + n], list(range(n)))]))
        at += n
        i += 1
    e.feed_close(r)
    return np.concatenate(outs)


def test_pages_and_slots_are_used_again(mix):
    """A pool of exactly two sequences' pages and two slots: later requests run in what earlier ones gave back, and a
    recurrent state (its matrix, its normaliser, its log-scale) starts from nothing in a slot that held another's."""
    cfg, W, d, o = mix
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


def test_a_step_over_the_pool_is_refused_and_leaves_the_engine_usable(mix):
    from kubeai_b200 import B200Error
    cfg, W, d, o = mix
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


# ---------------------------------------------------------------- edges made visible
QTOK, KTOK = 7, 11


def edge_model(tmp_path, softcap=None, q_temp=None, seed=31):
    """One layer whose attention copies from KTOK positions whenever a QTOK position can see one (planted pair, sharp
    softmax, an embedding large beside the position row)."""
    ty, mx = attention(heads=2, kv_heads=1, dim=32, vdim=16, scale=0.53, softcap=softcap, q_temp=q_temp, v_mix=False)
    cfg = make_config([dict(type=ty, mixer=mx, mlp=None)], width=48, vocab=40)
    W = plant_pair(cfg, random_weights(cfg, seed=seed, embed_gain=8.0), QTOK, KTOK)
    return cfg, W, write_model_dir(tmp_path / "edge", cfg, W)


def sequence_with(n, key_at, query_at, seed):
    """Random filler without the two special tokens, KTOK at key_at (None: nowhere), QTOK at query_at."""
    t = [x for x in np.random.default_rng(seed).integers(12, 40, size=n).tolist()]
    if key_at is not None:
        t[key_at] = KTOK
    t[query_at] = QTOK
    return t


@pytest.mark.parametrize("key_at,qpos", [(0, 300), (3, 410), (15, 200), (16, 200), (17, 81), (63, 130), (64, 130), (127, 129), (47, 48)])
def test_a_far_key_is_found_among_hundreds_and_across_page_borders(tmp_path, key_at, qpos):
    """One key, at the start of the sequence, on the last row of a page, on the first row of the next, or right before the
    query, decides the query's logits: the oracle's logits with and without it differ strongly, and the engine follows in
    a prompt step, in portions that cut between key and query, and token by token."""
    cfg, W, d = edge_model(tmp_path)
    o = oracle_for(cfg, W)
    with_key = sequence_with(qpos + 3, key_at, qpos, 1)
    without = sequence_with(qpos + 3, None, qpos, 1)
    w_with, w_without = o.forward(with_key), o.forward(without)
    assert rel_err(w_with[qpos:qpos + 1], w_without[qpos:qpos + 1])[0] > 0.3      # the key matters
    with open_engine(d) as e:
        close32(feed_whole(e, with_key), w_with)
        close32(feed_portions(e, with_key, [key_at + 1, 7, 1]), w_with)
        close32(feed_portions(e, with_key, [qpos - 2, 2, 1]), w_with)
        close32(feed_whole(e, without), w_without)
    with open_engine(d, dtype="bfloat16") as e:
        assert np.median(rel_err(feed_whole(e, with_key), w_with)) < 0.1
        assert rel_err(feed_portions(e, with_key, [qpos - 1, 1]), w_with)[qpos] < 0.25


@pytest.mark.parametrize("qpos", [5, 15, 16, 40, 63, 64])
def test_the_causal_edge_is_exact(tmp_path, qpos):
    """The key one position before the query decides its logits; the same key one position after it is invisible, in a
    prompt step (where it is in the same tile) and across a cut."""
    cfg, W, d = edge_model(tmp_path)
    o = oracle_for(cfg, W)
    before = sequence_with(qpos + 4, qpos - 1, qpos, 2)
    after = sequence_with(qpos + 4, qpos + 1, qpos, 2)
    w_before, w_after = o.forward(before), o.forward(after)
    assert rel_err(w_before[qpos:qpos + 1], w_after[qpos:qpos + 1])[0] > 0.3
    for dtype in ("float32", "bfloat16"):
        with open_engine(d, dtype=dtype) as e:
            for t, want in ((before, w_before), (after, w_after)):
                for got in (feed_whole(e, t), feed_portions(e, t, [qpos, 1, 3]), feed_portions(e, t, [qpos + 1, 1])):
                    if dtype == "float32":
                        close32(got, want)
                    else:
                        assert rel_err(got, want)[qpos] < 0.25


def test_capped_scores_bound_what_one_key_can_do(tmp_path):
    """With a cap far below the planted score the key no longer takes all the weight: the oracle's logits with and without
    the cap differ, and the engine follows the capped ones."""
    cfg, W, d = edge_model(tmp_path, softcap=2.0)
    free = dict(cfg, layers=[dict(cfg["layers"][0], mixer={k: v for k, v in cfg["layers"][0]["mixer"].items() if k != "softcap"})])
    t = sequence_with(120, 30, 110, 3)
    w_cap, w_free = oracle_for(cfg, W).forward(t), oracle_for(free, W).forward(t)
    assert rel_err(w_cap[110:111], w_free[110:111])[0] > 0.1
    with open_engine(d) as e:
        close32(feed_whole(e, t), w_cap)
        close32(feed_portions(e, t, [100, 1]), w_cap)


@pytest.mark.parametrize("every", [2, 16, 17, 33])
def test_the_query_gain_steps_at_the_right_positions(tmp_path, every):
    """The gain is constant up to position every - 2, steps at every - 1, and again one `every` later; with a strong
    coefficient the logits on both sides of a step differ from those of a model whose step lies one position later, in
    prompts, across cuts at the step, and token by token."""
    layers = [layer(attention(heads=2, kv_heads=1, dim=8, vdim=8, scale=1.2, q_temp=(3.0, every)), mlp=None)]
    cfg, W, d = build(tmp_path, layers, seed=33)
    later = make_config([layer(attention(heads=2, kv_heads=1, dim=8, vdim=8, scale=1.2, q_temp=(3.0, every + 1)), mlp=None)])
    t = toks(2 * every + 3, cfg["vocab"], 34)
    want, other = oracle_for(cfg, W).forward(t), oracle_for(later, W).forward(t)
    assert rel_err(want[every - 1:every], other[every - 1:every])[0] > 0.003 and rel_err(want[:every - 1], other[:every - 1]).max() == 0.0
    with open_engine(d) as e:
        close32(feed_whole(e, t), want)
        close32(feed_portions(e, t, [max(every - 1, 1), 1, 1, max(every - 2, 1), 1]), want)
        close32(feed_portions(e, t, [1]), want)


def test_far_tokens_reach_through_the_recurrent_state(tmp_path):
    """With forget gates close to one the matrix memory carries a token across hundreds of positions.  The first token is
    the one whose input gate is widest open and the rest are tokens whose gates are nearly shut, so that it still owns most
    of the state at the end: changing it changes the last logits, and the engine follows the oracle whether the prompt
    comes whole, in portions or decoded."""
    from oracle.mulenex_oracle import norm_one_plus, position_row
    cfg = make_config([layer(mlstm(heads=2, dim=8, vdim=8, gate_cap=12.0), mlp=None)])
    W = random_weights(cfg, seed=41, gate_bias=(-3.0, 9.0))
    W["l0.mix.i"] = W["l0.mix.i"] * 4.0
    d = write_model_dir(tmp_path / "m", cfg, W)
    o = oracle_for(cfg, W)
    cell = o.new_mixers()[0]
    x = W["embed"].astype(np.float64) + position_row(0, cfg["width"])
    gate = np.array([cell.gates(norm_one_plus(r, W["l0.norm1"].astype(np.float64), 1e-5))[0].min() for r in x])
    order = np.argsort(gate)
    quiet = order[:10]
    a = [int(order[-1])] + [int(quiet[i]) for i in np.random.default_rng(42).integers(0, 10, size=299)]
    b = [int(order[-2])] + a[1:]
    wa, wb = o.forward(a), o.forward(b)
    assert rel_err(wa[-1:], wb[-1:])[0] > 0.01
    with open_engine(d) as e:
        close32(feed_whole(e, a), wa, 3)
        close32(feed_portions(e, b, [150, 33, 1]), wb, 3)


@pytest.mark.parametrize("gate_bias", [(-7.0, 4.0), (5.0, 0.0), (0.0, 2.0)])
def test_first_tokens_of_a_sequence(tmp_path, gate_bias):
    """The log-scale of the recurrence starts at 0: with a weak input gate the first outputs rest on the floor e^(-m) of the
    denominator, with a strong one on |n . q|; the position row of position 0 is all cosines."""
    cfg, W, d = build(tmp_path, MIX, seed=52, gate_bias=gate_bias)
    o = oracle_for(cfg, W)
    with open_engine(d) as e:
        for n in (1, 2, 3):
            t = toks(n, cfg["vocab"], 50 + n)
            close32(feed_whole(e, t), o.forward(t))
        t = toks(6, cfg["vocab"], 54)
        close32(feed_portions(e, t, [1, 1, 2]), o.forward(t))


@pytest.mark.parametrize("seed", range(6))
def test_random_configurations(tmp_path, seed):
    rng = np.random.default_rng(100 + seed)
    layers, blend_shape = [], None
    for _ in range(int(rng.integers(1, 5))):
        if rng.random() < 0.55:
            G = int(rng.integers(1, 4))
            H = G * int(rng.integers(1, 4))
            vdim = int(rng.integers(1, 13))
            v_mix = rng.random() < 0.6
            if v_mix:
                if blend_shape is None:
                    blend_shape = (G, vdim)
                else:
                    H, G, vdim = H // G * blend_shape[0], blend_shape[0], blend_shape[1]
            mixer = attention(heads=H, kv_heads=G, dim=int(rng.integers(2, 13)), vdim=vdim, scale=float(rng.uniform(0.1, 0.9)),
                              softcap=None if rng.random() < 0.3 else float(rng.uniform(0.5, 30.0)),
                              q_temp=None if rng.random() < 0.3 else (float(rng.uniform(0.1, 2.0)), int(rng.integers(1, 40))), v_mix=v_mix)
        else:
            mixer = mlstm(heads=int(rng.integers(1, 4)), dim=int(rng.integers(1, 20)), vdim=int(rng.integers(1, 20)), gate_cap=float(rng.uniform(1.0, 20.0)))
        E = int(rng.integers(1, 9))
        u = rng.random()
        mlp = None if u < 0.25 else dense(ff=int(rng.integers(1, 30))) if u < 0.5 else \
            moe(experts=E, top=int(rng.integers(1, E + 1)), ff=int(rng.integers(1, 20)), shared=None if rng.random() < 0.4 else int(rng.integers(1, 20)))
        layers.append(layer(mixer, mlp=mlp))
    cfg, W, d = build(tmp_path, layers, seed=200 + seed, width=int(rng.integers(6, 40)), vocab=int(rng.integers(5, 60)),
                      gate_bias=(float(rng.uniform(-4, 4)), float(rng.uniform(-2, 6))))
    t = toks(70, cfg["vocab"], seed)
    want = oracle_for(cfg, W).forward(t)
    with open_engine(d) as e:
        close32(feed_whole(e, t), want, 3)
        close32(feed_portions(e, t, [int(rng.integers(2, 30)), int(rng.integers(1, 9)), 1]), want, 3)


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


def test_preemption_recomputes_cache_and_state_from_the_start(mix):
    """A pool too small for all running sequences to finish: the scheduler preempts and recomputes; outputs do not change."""
    cfg, W, d, o = mix
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
    cfg, W, d = build(tmp_path, MIX, seed=51, vocab=V)
    o = oracle_for(cfg, W)
    lim = default_config(manual_step=0, enable_prefix_caching=0, max_num_seqs=4, max_batched_tokens=32, max_model_len=256, num_kv_blocks=64)
    eng = Engine(lim, d, dtype="float32")
    srv = Server([eng], model="mx", vocab=V, max_model_len=256)
    try:
        out = {}

        def ask(i, text):
            body = dict(model="mx", messages=[{"role": "user", "content": text}], max_tokens=5, temperature=0, stream=(i == 0))
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
            prompt = srv.render_prompt("/v1/chat/completions", json.dumps(dict(model="mx", messages=[{"role": "user", "content": user}])))
            got = tokenize(text, V)
            assert len(got) == 5
            greedy_agrees(o, prompt, got)
    finally:
        srv.close()
        eng.close()


def test_a_checkpoint_without_a_tensor_the_config_asks_for_is_refused(tmp_path):
    from kubeai_b200 import B200Error
    from kubeai_b200.engine import Engine, default_config
    cfg = make_config([layer(mlstm())])
    short = random_weights(cfg)
    del short["l0.mix.f.b"]
    with pytest.raises(B200Error, match="f.b"):
        Engine(default_config(manual_step=1, max_model_len=64, num_kv_blocks=8), write_model_dir(tmp_path / "c", cfg, short), dtype="float32")


def test_blending_layers_of_different_value_shapes_are_refused(tmp_path):
    from kubeai_b200 import B200Error
    from kubeai_b200.engine import Engine, default_config
    cfg = make_config([layer(attention(vdim=6), mlp=None), layer(attention(vdim=8), mlp=None)])
    with pytest.raises(B200Error, match="blends"):
        Engine(default_config(manual_step=1), write_model_dir(tmp_path / "c", cfg, random_weights(cfg)), dtype="float32")
