"""Helpers for the Mulenex tests: small configurations, random bf16-representable weights (optionally with one planted
query/key pair whose score stands out), a model directory written from them, and the slow oracle over the same numbers."""
from __future__ import annotations

import numpy as np

from nomanex_util import bf16_round, feed_portions, feed_whole, open_engine, rel_err, write_model_dir  # noqa: F401  (re-exported)
from oracle.mulenex_oracle import MulenexOracle, norm_one_plus, position_row


def attention(heads=4, kv_heads=2, dim=8, vdim=6, scale=0.45, softcap=6.0, q_temp=(0.7, 5), v_mix=True):
    mx = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, v_mix=v_mix)
    if softcap:
        mx["softcap"] = softcap
    if q_temp:
        mx["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    return "attention", mx


def mlstm(heads=2, dim=6, vdim=10, gate_cap=9.0):
    return "mlstm", dict(heads=heads, dim=dim, vdim=vdim, gate_cap=gate_cap)


def dense(ff=20):
    return dict(kind="dense", ff=ff)


def moe(experts=5, top=2, ff=8, shared=12):
    m = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared:
        m["shared"] = dict(ff=shared)
    return m


def layer(mixer=None, mlp="default"):
    ty, mx = mixer or attention()
    return dict(type=ty, mixer=mx, mlp=moe() if mlp == "default" else mlp)


def make_config(layers, width=24, vocab=40, eps=1e-5):
    return dict(architecture="Mulenex", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)


def random_weights(cfg, seed=0, embed_gain=1.0, gate_bias=(0.0, 2.0), lam=None):
    """name -> float32 array whose values are exact in bfloat16.  gate_bias: means of the input- and forget-gate biases."""
    rng = np.random.default_rng(seed)
    Wd = cfg["width"]
    W = {}

    def mat(name, rows, cols, gain=1.0):
        W[name] = bf16_round(rng.standard_normal((rows, cols)).astype(np.float32) * gain / np.sqrt(cols))

    def vec(name, n, mean=0.0, spread=0.2):
        W[name] = bf16_round(mean + spread * rng.standard_normal(n).astype(np.float32))

    W["embed"] = bf16_round(rng.standard_normal((cfg["vocab"], Wd)).astype(np.float32) * embed_gain)
    mat("head", cfg["vocab"], Wd, 2.0)
    vec("final.norm", Wd)
    for i, ly in enumerate(cfg["layers"]):
        p, mx = "l%d." % i, ly["mixer"]
        for n in ("norm1", "norm1b"):
            vec(p + n, Wd)
        H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
        if ly["type"] == "attention":
            G = mx.get("kv_heads", H)
            mat(p + "mix.q", H * D, Wd, 2.0)
            mat(p + "mix.k", G * D, Wd, 2.0)
            mat(p + "mix.v", G * Dv, Wd, 2.0)
            mat(p + "mix.g", H, Wd, 3.0)
            mat(p + "mix.o", Wd, H * Dv, 2.0)
            vec(p + "mix.q.norm", D, 1.0)
            vec(p + "mix.k.norm", D, 1.0)
            W[p + "mix.vmix"] = bf16_round(np.array(rng.uniform(0.3, 0.7) if lam is None else lam, dtype=np.float32))
        else:
            mat(p + "mix.q", H * D, Wd, 2.0)
            mat(p + "mix.k", H * D, Wd, 2.0)
            mat(p + "mix.v", H * Dv, Wd, 2.0)
            mat(p + "mix.g", H * Dv, Wd, 2.0)
            mat(p + "mix.o", Wd, H * Dv, 2.0)
            vec(p + "mix.norm", H * Dv, 1.0)
            mat(p + "mix.i", H, Wd, 3.0)
            mat(p + "mix.f", H, Wd, 3.0)
            vec(p + "mix.i.b", H, gate_bias[0], 0.5)
            vec(p + "mix.f.b", H, gate_bias[1], 0.5)
        mlp = ly.get("mlp")
        if not mlp:
            continue
        for n in ("norm2", "norm2b"):
            vec(p + n, Wd)
        if mlp["kind"] == "dense":
            mat(p + "mlp.up", mlp["ff"], Wd, 2.0)
            mat(p + "mlp.down", Wd, mlp["ff"], 2.0)
            vec(p + "mlp.up.b", mlp["ff"], 0.0, 0.3)
            vec(p + "mlp.down.b", Wd, 0.0, 0.3)
            continue
        E = mlp["router"]["experts"]
        mat(p + "mlp.router", E, Wd, 3.0)
        vec(p + "mlp.router.b", E, 0.0, 0.5)
        for e in range(E):
            mat(p + "mlp.e%d.gate" % e, mlp["expert"]["ff"], Wd, 3.0)
            mat(p + "mlp.e%d.up" % e, mlp["expert"]["ff"], Wd, 3.0)
            mat(p + "mlp.e%d.down" % e, Wd, mlp["expert"]["ff"], 2.0)
        if mlp.get("shared"):
            mat(p + "mlp.shared.gate", mlp["shared"]["ff"], Wd, 3.0)
            mat(p + "mlp.shared.up", mlp["shared"]["ff"], Wd, 3.0)
            mat(p + "mlp.shared.down", Wd, mlp["shared"]["ff"], 2.0)
            mat(p + "mlp.shared.sg", 1, Wd, 3.0)
    return W


def plant_pair(cfg, W, query_token, key_token, layer=0, gain=6.0, post_boost=3.0):
    """Make the attention of `layer` (it must be the first layer, whose input is the token's embedding plus its position
    row) score key_token's key far above every other key for query_token's queries.  Every key head's projection gets a
    rank-one term q_dir sel^T: sel picks out key_token's normed input and is orthogonal to every other token's (taken at
    position 0; the embedding must be large beside the position row, and the vocabulary no larger than the width), q_dir
    points along query_token's normed and weighted query (first query head of the key head's group).  Keys are divided by
    their root mean square, so the planted key ends up parallel to that query whatever the gain, and with a sharp softmax
    (config scale) a query_token position copies the values of the visible key_token positions: its logits change
    visibly when one of them becomes invisible.  The weight of the norm behind the mixer is raised by post_boost, so that
    the mixer's output counts beside the large embedding."""
    mx = cfg["layers"][layer]["mixer"]
    H, G, D = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"]
    eps = cfg["norm"]["eps"]
    p = "l%d." % layer
    assert cfg["vocab"] <= cfg["width"]
    x = W["embed"].astype(np.float64) + position_row(0, cfg["width"])
    hs = norm_one_plus(x, W[p + "norm1"].astype(np.float64), eps)      # [vocab, width]
    pick = np.zeros(cfg["vocab"])
    pick[key_token] = 1.0
    sel = np.linalg.lstsq(hs, pick, rcond=None)[0]
    Wk = W[p + "mix.k"].astype(np.float64).reshape(G, D, -1)
    Wq = W[p + "mix.q"].astype(np.float64).reshape(H, D, -1)
    for g in range(G):
        q = Wq[g * (H // G)] @ hs[query_token]
        q = q * W[p + "mix.q.norm"].astype(np.float64) * W[p + "mix.k.norm"].astype(np.float64)
        Wk[g] += gain * np.linalg.norm(Wk[g] @ hs[key_token]) * np.outer(q / np.linalg.norm(q), sel)
    W[p + "mix.k"] = bf16_round(Wk.reshape(G * D, -1).astype(np.float32))
    W[p + "norm1b"] = bf16_round(W[p + "norm1b"] + post_boost)
    return W


def oracle_for(cfg, W):
    return MulenexOracle(cfg, W)
