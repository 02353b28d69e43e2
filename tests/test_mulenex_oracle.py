"""The Mulenex oracle's mechanisms against independent closed forms (CPU), the planted-pair construction the GPU tests
rely on, and the host-side configuration checks, which run before any device is touched."""
import math

import numpy as np
import pytest

from oracle import mulenex_oracle as O
from mulenex_util import attention, dense, layer, make_config, mlstm, moe, oracle_for, plant_pair, random_weights, rel_err


def sub(W, prefix):
    return {k[len(prefix):]: np.asarray(v, dtype=np.float64) for k, v in W.items() if k.startswith(prefix)}


def test_position_row_pairs_sine_and_cosine_of_one_angle():
    r0 = O.position_row(0, 6)
    assert np.array_equal(r0, [0, 1, 0, 1, 0, 1])
    r = O.position_row(3, 6)
    for i in range(3):
        ang = 3 * 10000.0 ** (-2.0 * i / 6)
        assert abs(r[2 * i] - math.sin(ang)) < 1e-15 and abs(r[2 * i + 1] - math.cos(ang)) < 1e-15
    odd = O.position_row(2, 5)          # an odd width ends on a sine
    assert abs(odd[4] - math.sin(2 * 10000.0 ** (-4.0 / 5))) < 1e-15


def test_norm_weight_is_an_offset_from_one():
    x = np.array([3.0, -4.0])
    assert np.allclose(O.norm_one_plus(x, np.zeros(2), 0.0), x / math.sqrt(12.5))
    assert np.allclose(O.norm_one_plus(x, np.array([1.0, -1.0]), 0.0), [2 * 3.0 / math.sqrt(12.5), 0.0])
    assert np.allclose(O.norm_one_plus(x, np.zeros(2), 12.5), x / 5.0)     # eps sits inside the root


def test_query_gain_steps_every_so_many_positions():
    qt = dict(coef=0.5, every=4)
    assert [O.query_gain(p, qt) for p in range(3)] == [1.0, 1.0, 1.0]
    assert O.query_gain(3, qt) == 1.0 + 0.5 * math.log(2) and O.query_gain(6, qt) == O.query_gain(3, qt)
    assert O.query_gain(7, qt) == 1.0 + 0.5 * math.log(3)
    assert O.query_gain(100, None) == 1.0


def test_matrix_memory_equals_the_unrolled_sums():
    """C_t e^(m_t) = sum_j exp(i_j + f_(j+1) + ... + f_t) k_j v_j^T: the stored state is that sum divided by e^(m_t), the
    denominator max(|n.q|, e^(-m)) + 1e-6 is taken in the stored scale, and m starts at 0."""
    cfg = make_config([layer(mlstm(heads=2, dim=5, vdim=4, gate_cap=3.0), mlp=None)], width=9)
    W = random_weights(cfg, seed=1, gate_bias=(-1.0, 0.5))
    P = sub(W, "l0.mix.")
    mx = cfg["layers"][0]["mixer"]
    hs = np.random.default_rng(2).standard_normal((12, 9)) * 2
    cell = O.MatrixMemory(P, mx, 1e-5)
    got = np.stack([cell.step(h) for h in hs])
    H, D, Dv, cap = 2, 5, 4, 3.0
    li = np.stack([cap * np.tanh((P["i"] @ h + P["i.b"]) / cap) for h in hs])
    lf = np.stack([-np.log1p(np.exp(-cap * np.tanh((P["f"] @ h + P["f.b"]) / cap))) for h in hs])
    for t in range(12):
        heads = []
        for a in range(H):
            m = 0.0
            for j in range(t + 1):
                m = max(lf[j, a] + m, li[j, a])
            C, n = np.zeros((D, Dv)), np.zeros(D)
            for j in range(t + 1):
                wgt = math.exp(li[j, a] + lf[j + 1:t + 1, a].sum())
                k = (P["k"] @ hs[j]).reshape(H, D)[a]
                C += wgt * np.outer(k, (P["v"] @ hs[j]).reshape(H, Dv)[a])
                n += wgt * k
            q = (P["q"] @ hs[t]).reshape(H, D)[a] / math.sqrt(D)
            heads.append((C.T @ q) * math.exp(-m) / (max(abs(n @ q) * math.exp(-m), math.exp(-m)) + 1e-6))
        y = np.concatenate([o / math.sqrt((o * o).mean() + 1e-5) for o in heads]) * P["norm"] * O.sigmoid(P["g"] @ hs[t])
        assert np.allclose(got[t], P["o"] @ y, rtol=1e-9, atol=1e-12)


def test_matrix_memory_log_scale_starts_at_zero_not_at_minus_infinity():
    """With a very negative input gate the first tokens keep m near 0 (decaying by f), and the output floor e^(-m) rules."""
    mx = dict(heads=1, dim=2, vdim=2, gate_cap=20.0)
    P = dict(q=np.eye(2), k=np.eye(2), v=np.eye(2), g=np.zeros((2, 2)), o=np.eye(2), norm=np.ones(2), i=np.zeros((1, 2)), f=np.zeros((1, 2)))
    P["i.b"], P["f.b"] = np.array([-8.0]), np.array([5.0])
    cell = O.MatrixMemory(P, mx, 1e-5)
    cell.step(np.array([1.0, 0.5]))
    lf = -math.log1p(math.exp(-20.0 * math.tanh(5.0 / 20.0)))
    assert abs(cell.m[0] - lf) < 1e-12 and cell.m[0] > -0.01        # m_1 = max(f + 0, i) = f, not i = -8


def test_attention_equals_dense_masked_attention():
    ty, mx = attention(heads=4, kv_heads=2, dim=6, vdim=5, scale=0.7, softcap=2.5, q_temp=(0.8, 3), v_mix=False)
    cfg = make_config([dict(type=ty, mixer=mx, mlp=None)], width=10)
    P = sub(random_weights(cfg, seed=3), "l0.mix.")
    hs = np.random.default_rng(4).standard_normal((11, 10))
    att = O.Attention(P, mx, 1e-5, None)
    got = np.stack([att.step(h) for h in hs])
    T, H, G, D, Dv = 11, 4, 2, 6, 5
    q = np.stack([O.unit_rms((P["q"] @ hs[t]).reshape(H, D), 1e-5) * P["q.norm"] * (1 + 0.8 * math.log((t + 1) // 3 + 1)) for t in range(T)])
    k = np.stack([O.unit_rms((P["k"] @ hs[t]).reshape(G, D), 1e-5) * P["k.norm"] for t in range(T)])
    v = np.stack([(P["v"] @ hs[t]).reshape(G, Dv) for t in range(T)])
    out = np.zeros((T, H * Dv))
    for a in range(H):
        s = 2.5 * np.tanh(q[:, a] @ k[:, a // 2].T * 0.7 / 2.5)
        s = np.where(np.tril(np.ones((T, T))) > 0, s, -np.inf)
        w = np.exp(s - s.max(-1, keepdims=True))
        w /= w.sum(-1, keepdims=True)
        out[:, a * Dv:(a + 1) * Dv] = (w @ v[:, a // 2]) * O.sigmoid(hs @ P["g"].T)[:, a:a + 1]
    assert np.allclose(got, out @ P["o"].T, rtol=1e-9, atol=1e-12)


def test_values_blend_with_the_first_blending_layers_values_only():
    """Layers: no blending, first blending layer (caches its own values), a blending layer (caches the blend), in between
    a recurrent layer.  With lambda = 1 the third attention caches exactly the second one's values."""
    layers = [layer(attention(v_mix=False), mlp=None), layer(attention(), mlp=None), layer(mlstm(), mlp=None), layer(attention(), mlp=None)]
    cfg = make_config(layers)
    W = random_weights(cfg, seed=5, lam=1.0)
    o = oracle_for(cfg, W)
    st = o.new_state()
    for t in (3, 9, 4):
        o.step(st, t)
    a0, a1, a3 = st["mixers"][0], st["mixers"][1], st["mixers"][3]
    assert a0.src is None and a1.src is None and a3.src is a1
    assert np.allclose(np.stack(a3.values), np.stack(a1.values))
    assert not np.allclose(np.stack(a3.values), np.stack(a0.values))
    W2 = dict(W)
    W2["l3.mix.vmix"] = np.float32(0.25)
    o2 = oracle_for(cfg, W2)
    st2 = o2.new_state()
    o2.step(st2, 3)
    b1, b3 = st2["mixers"][1], st2["mixers"][3]
    assert np.allclose(b3.values[0], 0.75 * b3.raw_value + 0.25 * b1.raw_value)


def test_routing_takes_the_largest_logits_and_weights_them_among_themselves():
    chosen, w = O.route(np.array([0.1, 2.0, -1.0, 2.0, 1.0]), 3)
    assert chosen == [1, 3, 4]                      # a tie goes to the lower index
    z = np.exp([2.0, 2.0, 1.0])
    assert np.allclose(w, z / z.sum())
    chosen, w = O.route(np.array([-50.0, -70.0]), 1)
    assert chosen == [0] and w[0] == 1.0            # negative logits rank as they are
    P = dict(router=np.eye(3), shared_unused=None)
    P["router.b"] = np.array([0.0, 0.0, 5.0])
    mlp = dict(router=dict(experts=3, top=1))
    for e in range(3):
        P["e%d.gate" % e] = np.full((1, 3), 10.0)
        P["e%d.up" % e] = np.full((1, 3), float(e + 1))
        P["e%d.down" % e] = np.ones((3, 1))
    h = np.array([1.0, 2.0, 0.0])
    y = O.moe_ff(P, mlp, h)                          # the bias makes expert 2 win over the larger plain logit of expert 1
    assert np.allclose(y, O.silu(30.0) * 9.0)


def test_dense_feed_forward_squares_the_rectified_biased_projection():
    P = dict(up=np.array([[1.0, 0.0], [0.0, 1.0]]), down=np.array([[1.0, 1.0]]))
    P["up.b"], P["down.b"] = np.array([0.5, -3.0]), np.array([0.25])
    assert np.allclose(O.dense_ff(P, np.array([1.5, 2.0])), [4.0 + 0.25])


def test_planted_pair_makes_one_key_decide():
    ty, mx = attention(heads=2, kv_heads=1, dim=32, vdim=16, scale=0.53, softcap=None, q_temp=None, v_mix=False)
    cfg = make_config([dict(type=ty, mixer=mx, mlp=None)], width=48, vocab=40)
    W = plant_pair(cfg, random_weights(cfg, seed=31, embed_gain=8.0), 7, 11)
    o = oracle_for(cfg, W)
    t = np.random.default_rng(1).integers(12, 40, size=60).tolist()
    t[50] = 7
    a, b = list(t), list(t)
    a[20] = 11
    b[51] = 11                                       # in the future of the query: invisible
    wa, wb, w0 = o.forward(a), o.forward(b), o.forward(t)
    assert rel_err(wa[50:51], w0[50:51])[0] > 0.3, rel_err(wa[50:51], w0[50:51])
    assert rel_err(wb[50:51], w0[50:51])[0] == 0.0


def test_generate_is_the_greedy_continuation():
    cfg = make_config([layer(), layer(mlstm(), mlp=dense())])
    o = oracle_for(cfg, random_weights(cfg, seed=6))
    out, margin = o.generate([1, 2, 3], 4)
    assert margin >= 0 and len(out) == 4
    assert out[0] == int(np.argmax(o.forward([1, 2, 3])[-1]))
    assert out[1] == int(np.argmax(o.forward([1, 2, 3, out[0]])[-1]))
