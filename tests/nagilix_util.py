"""Helpers for the Nagilix tests: small configurations, random bf16-representable weights (optionally with one planted
query/key pair whose score stands out), a model directory written from them, and the slow oracle over the same numbers."""
from __future__ import annotations

import numpy as np

from nomanex_util import bf16_round, feed_portions, feed_whole, open_engine, rel_err, write_model_dir  # noqa: F401  (re-exported)
from oracle.nagilix_oracle import NagilixOracle, unit_rms


def left(heads=4, kv_heads=2, dim=8, chunk=7, rot_dims=None, base=100.0, scale=0.4, conv=3):
    mx = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale)
    if conv:
        mx["conv"] = conv
    if chunk:
        mx["mask"] = dict(size=chunk)
    rd = dim // 2 * 2 if rot_dims is None else rot_dims
    if rd:
        mx["rot"] = dict(base=base, dims=rd)
    return mx


def right(heads=2, dim=8, vdim=6, decay=None, rot_dims=None, base=3000.0):
    mx = dict(heads=heads, dim=dim, vdim=vdim, decay=decay if decay is not None else [0.5 + 0.49 * i / max(heads - 1, 1) for i in range(heads)])
    rd = dim // 2 * 2 if rot_dims is None else rot_dims
    if rd:
        mx["rot"] = dict(base=base, dims=rd)
    return mx


def moe(experts=5, identity=2, top=2, ff=8, limit=1.5):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, identity=identity, top=top))


def parallel(l=None, r=None, mlp="default"):
    return dict(type="parallel", mixer=dict(left=l or left(), right=r or right()), mlp=moe() if mlp == "default" else mlp)


def mamba(inner=20, state=6, dt_rank=3, conv=4, mlp="default"):
    return dict(type="mamba1", mixer=dict(inner=inner, state=state, dt_rank=dt_rank, conv=conv), mlp=moe() if mlp == "default" else mlp)


def make_config(layers, width=24, vocab=40, streams=2, eps=1e-5, logit_scale=0.7, max_positions=512):
    cfg = dict(architecture="Nagilix", vocab=vocab, width=width, norm=dict(eps=eps), logit_scale=logit_scale, max_positions=max_positions,
               layers=layers)
    if streams is not None:
        cfg["streams"] = streams
    return cfg


def random_weights(cfg, seed=0, gated=True, pos_gain=0.3, left_only=False, right_only=False):
    """name -> float32 array whose values are exact in bfloat16.  left_only / right_only switch a parallel mixer's other
    branch off (its output weight 0), so that one branch alone decides the logits."""
    rng = np.random.default_rng(seed)
    Wd, ns = cfg["width"], cfg.get("streams")
    W = {}

    def mat(name, rows, cols, gain=1.0):
        W[name] = bf16_round(rng.standard_normal((rows, cols)).astype(np.float32) * gain / np.sqrt(cols))

    def vec(name, n, mean=1.0, dev=0.2):
        W[name] = bf16_round(mean + dev * rng.standard_normal(n).astype(np.float32))

    def one(name):
        W[name] = bf16_round(np.array(1.0 + 0.2 * rng.standard_normal(), dtype=np.float32))

    def hc(prefix):
        if not ns:
            return
        W[prefix + "in"] = bf16_round(1.0 / ns + 0.3 * rng.standard_normal(ns).astype(np.float32))
        W[prefix + "out"] = bf16_round(0.7 + 0.3 * rng.standard_normal(ns).astype(np.float32))
        W[prefix + "mix"] = bf16_round(np.eye(ns, dtype=np.float32) * 0.8 + 0.2 * rng.standard_normal((ns, ns)).astype(np.float32))

    def gate(prefix):
        if gated:
            mat(prefix, Wd, Wd, 2.0)
            vec(prefix + ".b", Wd, 0.5, 0.5)

    W["embed"] = bf16_round(rng.standard_normal((cfg["vocab"], Wd)).astype(np.float32))
    W["pos"] = bf16_round(pos_gain * rng.standard_normal((cfg["max_positions"], Wd)).astype(np.float32))
    mat("head", cfg["vocab"], Wd, 2.0)
    one("final.norm")
    for i, ly in enumerate(cfg["layers"]):
        p, mx = "l%d." % i, ly["mixer"]
        one(p + "norm1")
        hc(p + "hc1.")
        gate(p + "rg1")
        if ly["type"] == "parallel":
            l, r = mx["left"], mx["right"]
            H, G, D = l["heads"], l.get("kv_heads", l["heads"]), l["dim"]
            mat(p + "mix.left.q", H * D, Wd, 2.0)
            mat(p + "mix.left.k", G * D, Wd, 2.0)
            if l.get("conv", 1) > 1:
                W[p + "mix.left.q.conv"] = bf16_round(0.6 * rng.standard_normal((H * D, l["conv"])).astype(np.float32))
                W[p + "mix.left.k.conv"] = bf16_round(0.6 * rng.standard_normal((G * D, l["conv"])).astype(np.float32))
            vec(p + "mix.left.q.norm", H * D)
            vec(p + "mix.left.k.norm", G * D)
            vec(p + "mix.left.temp", H, 1.0, 0.3)
            vec(p + "mix.left.sink", H, 0.0, 1.0)
            mat(p + "mix.left.o", Wd, H * D, 2.0)
            Hr = r["heads"]
            mat(p + "mix.right.q", Hr * r["dim"], Wd, 2.0)
            mat(p + "mix.right.k", Hr * r["dim"], Wd, 2.0)
            mat(p + "mix.right.v", Hr * r["vdim"], Wd, 2.0)
            mat(p + "mix.right.g", Hr * r["vdim"], Wd, 2.0)
            mat(p + "mix.right.o", Wd, Hr * r["vdim"], 2.0)
            vec(p + "mix.left.out", Wd)
            vec(p + "mix.right.out", Wd)
            if left_only:
                W[p + "mix.right.out"][:] = 0.0
            if right_only:
                W[p + "mix.left.out"][:] = 0.0
        else:
            I, N, R = mx["inner"], mx["state"], mx["dt_rank"]
            mat(p + "mix.in", 2 * I, Wd, 2.0)
            W[p + "mix.conv"] = bf16_round(0.6 * rng.standard_normal((I, mx["conv"])).astype(np.float32))
            vec(p + "mix.conv.b", I, 0.0, 0.2)
            mat(p + "mix.x", R + 2 * N, I, 2.0)
            mat(p + "mix.dt", I, R, 1.5)
            vec(p + "mix.dt.b", I, -1.0, 1.0)
            W[p + "mix.A_log"] = bf16_round(np.log(rng.uniform(0.05, 4.0, size=(I, N))).astype(np.float32))
            vec(p + "mix.D", I)
            mat(p + "mix.o", Wd, I, 2.0)
        mlp = ly.get("mlp")
        if not mlp:
            continue
        one(p + "norm2")
        hc(p + "hc2.")
        gate(p + "rg2")
        ne = mlp["router"]["experts"] + mlp["router"].get("identity", 0)
        mat(p + "mlp.router", ne, Wd, 3.0)
        vec(p + "mlp.correction", ne, 0.0, 0.1)
        for e in range(mlp["router"]["experts"]):
            mat(p + "mlp.e%d.gate" % e, mlp["expert"]["ff"], Wd, 3.0)
            mat(p + "mlp.e%d.up" % e, mlp["expert"]["ff"], Wd, 3.0)
            mat(p + "mlp.e%d.down" % e, Wd, mlp["expert"]["ff"], 2.0)
    return W


def plant_pair(cfg, W, query_token, key_token, gain=8.0):
    """Make the left branch of layer 0 score key_token's key far above every other key for query_token's queries.

    The layer must have no convolution and no rotation, and the position rows must be zero, so that a token's key
    depends on the token alone.  Every key head's projection gets a rank-one term dir sel^T: sel picks out key_token's
    normed input and is orthogonal to every other token's (the vocabulary must not be larger than the width); dir points
    along the first query head's query of query_token, so the normed key of key_token is nearly parallel to that query
    and no other key is.  With a sharp softmax a query_token position then copies the values of the visible key_token
    positions, and its logits change visibly when such a position becomes invisible."""
    mx = cfg["layers"][0]["mixer"]["left"]
    H, G, D = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"]
    assert mx.get("conv", 1) <= 1 and not mx.get("rot") and cfg["vocab"] <= cfg["width"] and not np.any(W["pos"])
    eps, ns = cfg["norm"]["eps"], cfg.get("streams")
    x = W["embed"].astype(np.float64) * (W["l0.hc1.in"].astype(np.float64).sum() if ns else 1.0)
    hs = unit_rms(x, eps) * float(W["l0.norm1"])      # [vocab, width]
    pick = np.zeros(cfg["vocab"])
    pick[key_token] = 1.0
    sel = np.linalg.lstsq(hs, pick, rcond=None)[0]
    Wk = W["l0.mix.left.k"].astype(np.float64).reshape(G, D, -1)
    Wq = W["l0.mix.left.q"].astype(np.float64).reshape(H, D, -1)
    for g in range(G):
        q = Wq[g * (H // G)] @ hs[query_token]
        Wk[g] += gain * np.linalg.norm(Wk[g] @ hs[key_token]) * np.outer(q / np.linalg.norm(q), sel)
    W["l0.mix.left.k"] = bf16_round(Wk.reshape(G * D, -1).astype(np.float32))
    W["l0.mix.left.q.norm"][:] = 1.0
    W["l0.mix.left.k.norm"][:] = 1.0
    W["l0.mix.left.temp"][:] = 1.0
    return W


def oracle_for(cfg, W):
    return NagilixOracle(cfg, W)
