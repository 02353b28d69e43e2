"""The Nagilix oracle's mechanisms against independent closed forms (CPU), the planted-pair construction the GPU tests
rely on, and the host-side configuration checks, which run before any device is touched."""
import json

import numpy as np
import pytest

from oracle import nagilix_oracle as O
from nagilix_util import left, make_config, mamba, moe, oracle_for, parallel, plant_pair, random_weights, rel_err, right, write_model_dir


def test_rotation_pairs_a_dimension_with_the_one_half_the_span_further():
    rng = np.random.default_rng(0)
    rot = dict(dims=6, base=50.0)
    q, k = rng.standard_normal((1, 8)), rng.standard_normal((1, 8))
    a = (O.rotate_half(q, 11, rot) @ O.rotate_half(k, 4, rot).T).item()
    b = (O.rotate_half(q, 27, rot) @ O.rotate_half(k, 20, rot).T).item()
    assert abs(a - b) < 1e-9                                        # relative
    assert np.array_equal(O.rotate_half(q, 9, rot)[0, 6:], q[0, 6:])    # the tail passes unchanged
    r = O.rotate_half(np.array([[1.0, 0.0, 0.0, 0.0]]), 1, dict(dims=4, base=50.0))
    assert np.allclose(r, [[np.cos(1.0), 0.0, np.sin(1.0), 0.0]])    # entry 0 turns with entry 2, at frequency 1
    r = O.rotate_half(np.array([[0.0, 1.0, 0.0, 0.0]]), 2, dict(dims=4, base=49.0))
    assert np.allclose(r, [[0.0, np.cos(2.0 / 7.0), 0.0, np.sin(2.0 / 7.0)]])    # entry 1 with entry 3, at base^(-2/4)
    assert np.array_equal(O.rotate_half(q, 5, None), q)


def test_chunk_visibility_table():
    seen = [[j for j in range(9) if O.chunk_visible(i, j, 3)] for i in range(9)]
    assert seen[0] == [0] and seen[2] == [0, 1, 2] and seen[3] == [3] and seen[5] == [3, 4, 5] and seen[8] == [6, 7, 8]
    assert [j for j in range(6) if O.chunk_visible(4, j, None)] == [0, 1, 2, 3, 4]
    assert [j for j in range(6) if O.chunk_visible(4, j, 1)] == [4]


def test_sink_counts_once_in_the_denominator_and_has_no_value():
    s = np.array([0.3, -1.0, 2.0])
    w = O.sink_softmax(s, 0.5)
    full = np.exp(np.append(s, 0.5))
    assert np.allclose(w, (full / full.sum())[:3]) and w.sum() < 1.0
    assert np.allclose(O.sink_softmax(s, -1e9), np.exp(s) / np.exp(s).sum())
    assert O.sink_softmax(np.array([0.0]), 800.0)[0] == 0.0           # a huge sink takes everything, without overflow


def test_carried_convolution_equals_the_direct_sum():
    rng = np.random.default_rng(1)
    w, b, u = rng.standard_normal((3, 4)), rng.standard_normal(3), rng.standard_normal((9, 3))
    cv = O.CarriedConv(w, b)
    got = np.stack([cv.step(x) for x in u])
    for t in range(9):
        want = b + sum(w[:, j] * u[t - 3 + j] for j in range(4) if t - 3 + j >= 0)    # the last tap is the token's own
        assert np.abs(got[t] - want).max() < 1e-12
    one = O.CarriedConv(rng.standard_normal((3, 1)))
    assert np.allclose(one.step(u[0]), one.w[:, 0] * u[0])


def test_left_branch_equals_dense_chunked_attention_with_a_sink():
    cfg = make_config([parallel(l=left(heads=4, kv_heads=2, dim=6, chunk=4, rot_dims=4, conv=3), mlp=None)], width=10)
    W = {k: v.astype(np.float64) for k, v in random_weights(cfg, seed=1).items()}
    P = O.sub(W, "l0.mix.left.")
    mx = cfg["layers"][0]["mixer"]["left"]
    T, H, G, D = 11, 4, 2, 6
    hs = np.random.default_rng(2).standard_normal((T, 10))
    br = O.LeftBranch(P, mx, 1e-5)
    got = np.stack([br.step(h) for h in hs])

    def conv(u, w):
        pad = np.concatenate([np.zeros((w.shape[1] - 1, u.shape[1])), u])
        return sum(w[:, j] * pad[j:j + len(u)] for j in range(w.shape[1]))

    q, k = conv(hs @ P["q"].T, P["q.conv"]), conv(hs @ P["k"].T, P["k.conv"])
    v = k.reshape(T, G, D)
    q = q / np.sqrt((q * q).mean(-1, keepdims=True) + 1e-5) * P["q.norm"]      # over all heads at once
    k = k / np.sqrt((k * k).mean(-1, keepdims=True) + 1e-5) * P["k.norm"]
    q = np.stack([O.rotate_half(q[t].reshape(H, D), t, mx["rot"]) for t in range(T)])
    k = np.stack([O.rotate_half(k[t].reshape(G, D), t, mx["rot"]) for t in range(T)])
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    vis = (j <= i) & (i // 4 == j // 4)
    out = np.zeros((T, H, D))
    for h in range(H):
        s = np.where(vis, q[:, h] @ k[:, h // 2].T * mx["scale"] * P["temp"][h], -np.inf)
        e = np.exp(s)
        out[:, h] = e / (e.sum(-1, keepdims=True) + np.exp(P["sink"][h])) @ v[:, h // 2]
    assert np.abs(got - out.reshape(T, -1) @ P["o"].T).max() < 1e-10


def test_right_branch_equals_the_unrolled_decay_sum():
    cfg = make_config([parallel(r=right(heads=2, dim=4, vdim=3, decay=[0.5, 0.9], rot_dims=2), mlp=None)], width=6)
    W = {k: v.astype(np.float64) for k, v in random_weights(cfg, seed=3).items()}
    P = O.sub(W, "l0.mix.right.")
    mx = cfg["layers"][0]["mixer"]["right"]
    hs = np.random.default_rng(4).standard_normal((7, 6))
    br = O.RightBranch(P, mx, 1e-5)
    got = np.stack([br.step(h) for h in hs])
    q = np.stack([O.rotate_half((P["q"] @ hs[t]).reshape(2, 4), t, mx["rot"]) for t in range(7)])
    k = np.stack([O.rotate_half((P["k"] @ hs[t]).reshape(2, 4), t, mx["rot"]) for t in range(7)]) / 2.0      # dim^(-1/2)
    v = (hs @ P["v"].T).reshape(7, 2, 3)
    for t in range(7):
        o = np.stack([sum(mx["decay"][h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1)) for h in range(2)])
        o = o / np.sqrt((o * o).mean(-1, keepdims=True) + 1e-5)              # every head by its own root mean square
        want = P["o"] @ (o.reshape(-1) * O.silu(P["g"] @ hs[t]))
        assert np.abs(got[t] - want).max() < 1e-10


def test_selective_scan_equals_the_unrolled_sum():
    cfg = make_config([mamba(inner=5, state=3, dt_rank=2, conv=2, mlp=None)], width=6)
    W = {k: v.astype(np.float64) for k, v in random_weights(cfg, seed=5).items()}
    P = O.sub(W, "l0.mix.")
    hs = np.random.default_rng(6).standard_normal((6, 6))
    mm = O.MambaMixer(P, cfg["layers"][0]["mixer"], 1e-5)
    got = np.stack([mm.step(h) for h in hs])
    xz = hs @ P["in"].T
    xin, z = xz[:, :5], xz[:, 5:]
    x = np.stack([P["conv.b"] + P["conv"][:, 1] * xin[t] + (P["conv"][:, 0] * xin[t - 1] if t else 0.0) for t in range(6)])
    x = x / (1.0 + np.exp(-x))
    low = x @ P["x"].T
    d = np.log1p(np.exp(low[:, :2] @ P["dt"].T + P["dt.b"]))
    B, C, A = low[:, 2:5], low[:, 5:], -np.exp(P["A_log"])
    for t in range(6):
        # S_t = sum_j exp(A * (d_(j+1) + ... + d_t)) d_j x_j B_j
        S = sum(np.exp(A * d[j + 1:t + 1].sum(0)[:, None]) * (d[j] * x[j])[:, None] * B[j][None, :] for j in range(t + 1))
        want = P["o"] @ ((S @ C[t] + P["D"] * x[t]) * O.silu(z[t]))
        assert np.abs(got[t] - want).max() < 1e-10


def test_router_ranks_with_the_correction_weights_without_it_and_knows_identity_experts():
    P = dict(router=np.array([[2.0, 0.0], [0.0, 2.0], [1.0, 1.0], [-1.0, 0.0]]), correction=np.array([0.0, 0.0, 0.0, 0.9]))
    h = np.array([1.0, 0.2])
    z = P["router"] @ h
    s = np.exp(z) / np.exp(z).sum()
    chosen, weights, margin = O.route(P, h, dict(experts=3, identity=1, top=2))
    assert chosen == [3, 0]                      # the correction lifts the last output over everything
    assert np.allclose(weights, [s[3], s[0]]) and sum(weights) < 1.0      # the chosen scores are the weights as they are: they need not sum to one
    assert abs(margin - (s[0] - s[2])) < 1e-12
    P.update({"e0.gate": np.array([[1.0, 0.0]]), "e0.up": np.array([[0.0, 5.0]]), "e0.down": np.array([[1.0], [2.0]])})
    y = O.moe_ff(P, dict(router=dict(experts=3, identity=1, top=2), expert=dict(limit=0.8)), h)
    g, u = min(1.0, 0.8), min(1.0, 0.8)
    want = s[3] * h + s[0] * np.array([1.0, 2.0]) * (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0))     # output 3 is the identity expert
    assert np.abs(y - want).max() < 1e-12


def test_streams_read_and_write():
    rng = np.random.default_rng(7)
    xs = [rng.standard_normal(5) for _ in range(3)]
    y = rng.standard_normal(5)
    hc = dict(mix=rng.standard_normal((3, 3)), out=rng.standard_normal(3))
    hc["in"] = rng.standard_normal(3)
    assert np.allclose(O.streams_read(xs, hc), hc["in"][0] * xs[0] + hc["in"][1] * xs[1] + hc["in"][2] * xs[2])
    assert np.allclose(np.stack(O.streams_write(xs, hc, y)), hc["mix"].T @ np.stack(xs) + np.outer(hc["out"], y))      # mix is indexed [from, to]
    one = O.streams_write([xs[0]], None, y)
    assert len(one) == 1 and np.allclose(one[0], xs[0] + y)


def test_the_write_back_is_gated_by_the_sublayers_own_input():
    cfg = make_config([parallel(mlp=None)], streams=None)
    W = random_weights(cfg, seed=8)
    o = oracle_for(cfg, W)
    shut = dict(W)
    shut["l0.rg1.b"] = np.full_like(W["l0.rg1.b"], -80.0)        # sigmoid(-80 + ...) = 0: the sublayer writes nothing back
    lg = oracle_for(cfg, shut).forward([3, 5, 7])
    x = (W["embed"][[3, 5, 7]] + W["pos"][:3]).astype(np.float64)
    want = (O.unit_rms(x, 1e-5) * float(W["final.norm"])) @ W["head"].astype(np.float64).T * cfg["logit_scale"]
    assert np.abs(lg - want).max() < 1e-9
    assert np.abs(o.forward([3, 5, 7]) - want).max() > 1e-2


def test_planted_pair_makes_one_key_decide():
    cfg = make_config([parallel(l=left(heads=2, kv_heads=1, dim=16, chunk=9, rot_dims=0, scale=6.0, conv=0), mlp=None)], width=48, vocab=40)
    W = plant_pair(cfg, random_weights(cfg, seed=31, pos_gain=0.0, left_only=True), 7, 11)
    o = oracle_for(cfg, W)
    base = np.random.default_rng(1).integers(12, 40, size=30).tolist()
    base[26] = 7                             # chunk [18, 27)
    a, b = list(base), list(base)
    a[18], b[17] = 11, 11                    # the chunk's first position; the last position of the chunk before
    assert rel_err(o.forward(a)[26:27], o.forward(b)[26:27])[0] > 0.3


def test_config_errors_come_before_any_device_work(tmp_path):
    from kubeai_b200 import B200Error
    from kubeai_b200.engine import Engine, default_config
    cfg = make_config([parallel(), mamba()])
    W = random_weights(cfg)
    lim = default_config(manual_step=1)
    for i, (edit, msg) in enumerate([
            (lambda c: c["layers"][0].update(type="serial"), "unknown mixer"),
            (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
            (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=5), "values from the keys"),
            (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5]), "decay"),
            (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
            (lambda c: c["layers"][1]["mixer"].pop("state"), "state"),
            (lambda c: c.pop("max_positions"), "max_positions"),
            (lambda c: c.update(streams=9), "streams")]):
        bad = json.loads(json.dumps(cfg))
        edit(bad)
        with pytest.raises(B200Error, match=msg):
            Engine(lim, write_model_dir(tmp_path / ("b%d" % i), bad, W), dtype="float32")
