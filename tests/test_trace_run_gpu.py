"""bin/trace_run as a user runs it: a model directory, a schedule of steps on standard input, logits files out.  The
schedule mixes prompt portions with single tokens, holds at most four requests at a time in a pool sized for them, and
admits a fifth request into the pages and the slot a finished one gave back; the logits are the oracle's."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import mulenex_util as mx
import nagilix_util as nx
from zinavik_util import layer, left, make_config, moe, oracle_for, random_weights, rel_err, right, write_model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def schedule(seqs):
    """Steps as the runner reads them, and for every step the (request, positions) its logits belong to."""
    plan = {"a": [40, 3, 1, 1, 30, 1, 2], "b": [1, 1, 17, 2, 1], "c": [64, 7], "d": [2, 2, 2, 1], "e": [0, 0, 0, 0, 0, 0, 0, 33, 5, 1]}
    at = {k: 0 for k in seqs}
    steps, rows, n = [], [], 0
    while any(at[k] < len(seqs[k]) for k in seqs):
        entries, end, want = [], [], []
        for k in seqs:
            p = plan[k]
            cnt = p[n] if n < len(p) else 1
            cnt = min(cnt, len(seqs[k]) - at[k])
            if cnt <= 0:
                continue
            pick = [i for i in range(cnt) if (at[k] + i) % 3 != 1]
            entries.append({"id": k, "tokens": seqs[k][at[k]:at[k] + cnt], "want": pick})
            want += [(k, at[k] + i) for i in pick]
            at[k] += cnt
            if at[k] == len(seqs[k]):
                end.append(k)
        steps.append(json.dumps({"step": n, "entries": entries, "end": end}))
        rows.append(want)
        n += 1
    return steps, rows


def zinavik_model():
    layers = [layer(l=left(heads=6, kv_heads=3, dim=16, vdim=16, window=21, keep_first=5), r=right(heads=2, dim=12, vdim=20), mlp=moe(experts=4, top=4, ff=24, shared=8)),
              layer(l=left(heads=2, kv_heads=2, dim=8, vdim=4, window=50, keep_first=0, rot_dims=4, scaling=None), mlp=None)]
    cfg = make_config(layers, width=40, vocab=70, streams=3, loop=(0, 1, 2))
    W = random_weights(cfg, seed=91)
    return cfg, W, oracle_for(cfg, W)


def mulenex_model():
    layers = [mx.layer(mx.attention(heads=6, kv_heads=3, dim=16, vdim=16, q_temp=(0.8, 7)), mlp=mx.moe(experts=4, top=4, ff=24, shared=8)),
              mx.layer(mx.mlstm(heads=2, dim=12, vdim=20), mlp=mx.dense(ff=48)), mx.layer(mx.attention(heads=3, kv_heads=3, dim=8, vdim=16, softcap=None), mlp=None)]
    cfg = mx.make_config(layers, width=40, vocab=70)
    W = mx.random_weights(cfg, seed=93)
    return cfg, W, mx.oracle_for(cfg, W)


def nagilix_model():
    layers = [nx.parallel(l=nx.left(heads=6, kv_heads=3, dim=16, chunk=21, conv=4), r=nx.right(heads=2, dim=12, vdim=20), mlp=nx.moe(experts=3, identity=1, top=4, ff=24)),
              nx.mamba(inner=48, state=8, dt_rank=4, mlp=None), nx.parallel(l=nx.left(heads=2, kv_heads=2, dim=8, chunk=50, rot_dims=4, conv=2), mlp=None)]
    cfg = nx.make_config(layers, width=40, vocab=70, streams=3)
    W = nx.random_weights(cfg, seed=95)
    return cfg, W, nx.oracle_for(cfg, W)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("model", [zinavik_model, mulenex_model, nagilix_model])
def test_replayed_schedule_gives_the_oracles_logits(tmp_path, dtype, model):
    cfg, W, o = model()
    d = write_model_dir(tmp_path / "m", cfg, W)
    rng = np.random.default_rng(92)
    seqs = {k: rng.integers(0, 70, size=n).tolist() for k, n in (("a", 90), ("b", 31), ("c", 71), ("d", 7), ("e", 45))}
    steps, rows = schedule(seqs)
    out = tmp_path / "out"
    # a, b, c, d live together: 96 + 32 + 80 + 16 tokens of pages; e comes when d and b are gone
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out), "--max-tokens", "256"],
                       input="\n".join(steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.splitlines() if ln.startswith("done ")] == ["done %d" % i for i in range(len(steps))]
    want = {k: o.forward(seqs[k]) for k in seqs}
    errs = []
    for n, r in enumerate(rows):
        f = out / ("%d.f32" % n)
        if not r:
            assert not f.exists()
            continue
        got = np.fromfile(f, dtype="<f4").reshape(len(r), 70)
        errs.append(rel_err(got, np.stack([want[k][pos] for k, pos in r])))
    errs = np.concatenate(errs)
    if dtype == "float32":
        assert np.median(errs) < 2e-5 and errs.max() < 3e-4
    else:
        assert np.median(errs) < 0.06 and np.quantile(errs, 0.9) < 0.2
