"""Prefill and decode throughput of a registered design beside the closest existing model at equal width, depth, head
and feed-forward sizes, on random weights (`bench.py --design nomanex`: beside the built-in Llama model;
`bench.py --design zinavik`: beside Nomanex, whose recurrent scan, windowed attention and routed experts are the like
kernels; `bench.py --design mulenex`: beside Zinavik, which runs the same attention, scan, routing and projection kernels;
`bench.py --design nagilix`: beside Zinavik, whose streams, paged attention, constant-decay scan and clamped routed experts
are the like kernels).  Every number is CUDA-event time of the engine's
own step (b200_feed_step: the same packing, page pool, state slots and kernels as a scheduled step), after warm-up
steps, with a buffer larger than L2 written between timed steps.  Per-kernel times come from a separate pass in which
each launch is bracketed by events (b200_engine_profile_kernels for the design, b200_engine_profile_range for Llama),
and are turned into fractions of the measured bf16 / HBM peaks from the kernels' algorithmic FLOPs and bytes."""
from __future__ import annotations

import json
import os
import tempfile

import numpy as np

SIZES = {
    # name: width, latent/gla heads, dense ff, experts x expert ff (top, groups, keep), window, layers of each kind
    "w2048": dict(width=2048, heads=16, ff=8192, experts=16, eff=2048, top=2, groups=4, keep=2, window=1024, vocab=32000),
    "w4096": dict(width=4096, heads=32, ff=14336, experts=16, eff=4096, top=2, groups=4, keep=2, window=2048, vocab=32000),
}
DIM, ROT, VDIM, RANK = 128, 64, 128, 512


def nomanex_config(z):
    lat = dict(heads=z["heads"], dim=DIM, rot_dim=ROT, vdim=VDIM, kv_rank=RANK, mask=dict(size=z["window"]),
               rot=dict(base=10000.0, dims=ROT), scale=(DIM + ROT) ** -0.5)
    gl = dict(heads=z["heads"], dim=DIM, vdim=VDIM, tau=16.0)
    dn = dict(kind="dense", ff=z["ff"], limit=7.0)
    mo = dict(kind="moe", expert=dict(ff=z["eff"]), router=dict(experts=z["experts"], top=z["top"], groups=dict(count=z["groups"], keep=z["keep"])))
    layers = [dict(type="latent_attention", mixer=lat, mlp=dn), dict(type="gla", mixer=gl, mlp=mo),
              dict(type="gla", mixer=gl, mlp=dn), dict(type="latent_attention", mixer=lat, mlp=mo)]
    return dict(architecture="Nomanex", vocab=z["vocab"], width=z["width"], residual_mult=0.5, norm=dict(eps=1e-5),
                embedding=dict(bigram=dict(buckets=65521, mul_prev=127, mul_cur=17)), layers=layers)


def zinavik_config(z):
    H = z["heads"]
    lf = dict(heads=H, kv_heads=max(1, H // 4), dim=DIM, vdim=VDIM, mask=dict(size=z["window"], keep_first=4),
              rot=dict(base=10000.0, dims=ROT, scaling=dict(factor=4.0, original=2048, fast=32.0, slow=1.0)), scale=DIM ** -0.5)
    rt = dict(heads=H, dim=DIM, vdim=VDIM, decay=[1.0 - 2.0 ** -(5.0 + 5.0 * h / max(H - 1, 1)) for h in range(H)])
    mo = dict(kind="moe", expert=dict(ff=z["eff"], limit=7.0), router=dict(experts=z["experts"], top=z["top"]),
              shared=dict(ff=z["eff"], limit=7.0))
    ly = dict(type="parallel", mixer=dict(left=lf, right=rt, left_scale=1.0, right_scale=1.0), mlp=mo)
    return dict(architecture="Zinavik", vocab=z["vocab"], width=z["width"], norm=dict(eps=1e-5), embedding=dict(scale=1.0), streams=2,
                layers=[ly, ly, ly, ly])


def mulenex_config(z):
    H = z["heads"]
    at = dict(heads=H, kv_heads=max(1, H // 4), dim=DIM, vdim=VDIM, scale=DIM ** -0.5, softcap=30.0, q_temp=dict(coef=0.1, every=256), v_mix=True)
    ml = dict(heads=H, dim=DIM, vdim=VDIM, gate_cap=15.0)
    mo = dict(kind="moe", expert=dict(ff=z["eff"]), router=dict(experts=z["experts"], top=z["top"]), shared=dict(ff=z["eff"]))
    dn = dict(kind="dense", ff=z["ff"])
    layers = [dict(type="attention", mixer=at, mlp=mo), dict(type="mlstm", mixer=ml, mlp=mo),
              dict(type="attention", mixer=at, mlp=dn), dict(type="mlstm", mixer=ml, mlp=mo)]
    return dict(architecture="Mulenex", vocab=z["vocab"], width=z["width"], norm=dict(eps=1e-5), layers=layers)


def nagilix_config(z):
    H, W = z["heads"], z["width"]
    lf = dict(heads=H, kv_heads=max(1, H // 4), dim=DIM, vdim=DIM, conv=4, mask=dict(size=z["window"]), rot=dict(base=10000.0, dims=ROT), scale=DIM ** -0.5)
    rt = dict(heads=H, dim=DIM, vdim=VDIM, decay=[1.0 - 2.0 ** -(5.0 + 5.0 * h / max(H - 1, 1)) for h in range(H)], rot=dict(base=10000.0, dims=DIM))
    mo = dict(kind="moe", expert=dict(ff=z["eff"], limit=7.0), router=dict(experts=z["experts"], identity=2, top=z["top"]))
    pa = dict(type="parallel", mixer=dict(left=lf, right=rt), mlp=mo)
    ma = dict(type="mamba1", mixer=dict(inner=2 * W, state=16, dt_rank=W // 16, conv=4), mlp=mo)
    return dict(architecture="Nagilix", vocab=z["vocab"], width=W, norm=dict(eps=1e-5), logit_scale=1.0, max_positions=4096, streams=2,
                layers=[pa, ma, pa, ma])


def flush_l2(torch, buf):
    buf.add_(1)
    torch.cuda.synchronize()


def run_engine(e, torch, buf, vocab, batch, prompt, decode_steps, warmup):
    rng = np.random.default_rng(0)
    out = {}
    # prefill: `batch` prompts of `prompt` tokens in one step
    times = []
    for it in range(warmup + 3):
        rids = [e.feed_open() for _ in range(batch)]
        flush_l2(torch, buf)
        e.feed_step([(r, rng.integers(0, vocab, size=prompt).tolist(), [prompt - 1]) for r in rids])
        times.append(e.stats().last_step_device_us)
        if it < warmup + 2:
            for r in rids:
                e.feed_close(r)
    us = float(np.median(times[warmup:]))
    out["prefill"] = dict(tokens=batch * prompt, step_ms=us / 1e3, tok_s=batch * prompt / us * 1e6)
    # decode: the last batch stays live; one token per sequence per step
    times = []
    for it in range(warmup + decode_steps):
        flush_l2(torch, buf)
        e.feed_step([(r, [int(rng.integers(0, vocab))], [0]) for r in rids])
        times.append(e.stats().last_step_device_us)
    us = float(np.median(times[warmup:]))
    out["decode"] = dict(seqs=batch, context=prompt + warmup, step_ms=us / 1e3, tok_s=batch / us * 1e6)
    return out, rids


def run_design(cfgj, lim, z, batch, prompt, decode_steps, warmup, peaks, torch, buf):
    """One registered design on random weights: step times, per-kernel times and fractions of the measured peaks."""
    from .engine import Engine, default_config
    hbm, tf, _ = peaks
    T = batch * prompt
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfgj, f)
        with Engine(default_config(**lim), d, dtype="bfloat16", random_weights=True) as e:
            r, rids = run_engine(e, torch, buf, z["vocab"], batch, prompt, decode_steps, warmup)
            # per-kernel pass: one prefill step of the same shape, then one decode step
            for q in rids:
                e.feed_close(q)
            rng = np.random.default_rng(1)
            rids = [e.feed_open() for _ in range(batch)]
            e.profile_kernels(True)
            e.feed_step([(q, rng.integers(0, z["vocab"], size=prompt).tolist(), [prompt - 1]) for q in rids])
            kp = e.kernel_times()
            e.profile_kernels(True)
            e.feed_step([(q, [1], [0]) for q in rids])
            kd = e.kernel_times()
            e.profile_kernels(False)
            r["kernels_prefill_us"] = {k: round(v["us"], 1) for k, v in sorted(kp.items())}
            r["kernels_decode_us"] = {k: round(v["us"], 1) for k, v in sorted(kd.items())}
            H, W = z["heads"], z["width"]
            us = lambda k, name: k[name]["us"] * 1e-6
            if cfgj["architecture"] == "Nomanex":
                # algorithmic work of the two mixers and of the projections (per step, both layers of a kind together)
                E = RANK + ROT
                keys = sum(min(p + 1, z["window"]) for p in range(prompt)) * batch
                att_flops = 2.0 * 2 * H * keys * (E + RANK)
                gla_flops = 2.0 * 3 * 2 * T * H * DIM * VDIM
                n_in = sum(_n_in(ly, W) for ly in cfgj["layers"])
                k_out = sum(_k_out(ly) for ly in cfgj["layers"])
                proj_flops = 2.0 * T * W * (n_in + k_out)
                state_bytes = 2.0 * 2 * batch * H * DIM * VDIM * 4
                dkeys = batch * min(prompt + 1, z["window"])
                nl = len(cfgj["layers"]) + 1
                r["roofline"] = {
                    "latent_attention_prefill_frac_of_bf16_peak": att_flops / us(kp, "latent_attention") / (tf * 1e12),
                    "gla_scan_prefill_tflops": gla_flops / us(kp, "gla_scan") / 1e12,
                    "projections_prefill_frac_of_bf16_peak": proj_flops / (us(kp, "proj_in") + us(kp, "proj_out")) / (tf * 1e12),
                    "gla_scan_decode_frac_of_hbm": state_bytes / us(kd, "gla_scan") / (hbm * 1e9),
                    "latent_attention_decode_frac_of_hbm": 2.0 * dkeys * E * 2 / us(kd, "latent_attention") / (hbm * 1e9),
                    "projections_decode_frac_of_hbm": 2.0 * W * (n_in + k_out) / (us(kd, "proj_in") + us(kd, "proj_out")) / (hbm * 1e9),
                    # residual update + norm: reads the fp32 residual and two bf16 sublayer outputs, writes the residual and a bf16 row
                    "residual_norm_prefill_frac_of_hbm": nl * T * W * (4 + 4 + 2 + 2 + 2) / us(kp, "residual_norm") / (hbm * 1e9),
                    "moe_experts_prefill_frac_of_bf16_peak": 2.0 * 2 * T * z["top"] * 2 * W * z["eff"] / (us(kp, "moe_up") + us(kp, "moe_down")) / (tf * 1e12),
                }
            elif cfgj["architecture"] == "Nagilix":
                par = [ly for ly in cfgj["layers"] if ly["type"] == "parallel"]
                mam = [ly for ly in cfgj["layers"] if ly["type"] == "mamba1"]
                L, Lp, Lm = len(cfgj["layers"]), len(par), len(mam)
                lf, mm = par[0]["mixer"]["left"], mam[0]["mixer"]
                G, ns, chunk = lf["kv_heads"], cfgj["streams"], lf["mask"]["size"]
                I, N, R = mm["inner"], mm["state"], mm["dt_rank"]
                keys = sum(p % chunk + 1 for p in range(prompt)) * batch
                att_flops = 2.0 * Lp * H * keys * (DIM + DIM)
                scan_flops = 2.0 * 3 * Lp * T * H * DIM * VDIM
                n_in = Lp * (H * DIM + G * DIM + 2 * H * DIM + 2 * H * VDIM + W) + Lm * (2 * I + W)
                k_out = Lp * (H * DIM + H * VDIM) + Lm * I
                proj_flops = 2.0 * T * W * (n_in + k_out + L * W)       # the feed-forward's gate projection counts among them
                pk = lambda k: us(k, "proj_in") + us(k, "proj_out") + us(k, "proj_gate")
                dkeys = batch * (prompt % chunk + 1)
                calls = 2 * L + 1
                r["roofline"] = {
                    "chunk_attention_prefill_frac_of_bf16_peak": att_flops / us(kp, "chunk_attention") / (tf * 1e12),
                    "retention_scan_prefill_tflops": scan_flops / us(kp, "retention_scan") / 1e12,
                    "projections_prefill_frac_of_bf16_peak": proj_flops / pk(kp) / (tf * 1e12),
                    "retention_scan_decode_frac_of_hbm": 2.0 * Lp * batch * H * DIM * VDIM * 4 / us(kd, "retention_scan") / (hbm * 1e9),
                    "chunk_attention_decode_frac_of_hbm": Lp * dkeys * G * 2 * DIM * 2.0 / us(kd, "chunk_attention") / (hbm * 1e9),
                    "projections_decode_frac_of_hbm": 2.0 * W * (n_in + k_out + L * W) / pk(kd) / (hbm * 1e9),
                    # stream boundary: reads and writes `ns` fp32 streams, reads a sublayer output and its gate row, writes a bf16 row
                    "stream_norm_prefill_frac_of_hbm": calls * T * W * (8.0 * ns + 2 + 2 + 2) / us(kp, "stream_norm") / (hbm * 1e9),
                    "moe_experts_prefill_frac_of_bf16_peak": 2.0 * L * T * z["top"] * 3 * W * z["eff"] / (us(kp, "moe_up") + us(kp, "moe_down")) / (tf * 1e12),
                    # selective scan: per (token, channel, state) one exponential and two multiply-adds; the step reads x, z, the
                    # fp32 step sizes and writes y; a decode step reads and writes every sequence's state once
                    "selective_scan_prefill_gelem_s": Lm * T * I * N / us(kp, "selective_scan") / 1e9,
                    "selective_scan_prefill_frac_of_hbm": Lm * T * I * (2 + 2 + 4 + 2.0) / us(kp, "selective_scan") / (hbm * 1e9),
                    "selective_scan_decode_frac_of_hbm": 2.0 * Lm * batch * I * N * 4 / us(kd, "selective_scan") / (hbm * 1e9),
                    # the preparation of the chunked attention: reads q | k rows (and taps - 1 rows before), writes fp32 queries and the cache row
                    "conv_qk_prep_prefill_frac_of_hbm": Lp * T * ((H + G) * DIM * 2.0 + H * DIM * 4 + 2 * G * DIM * 2) / us(kp, "conv_qk_prep") / (hbm * 1e9),
                    "short_conv_prefill_frac_of_hbm": Lm * T * I * (2.0 + 2) / us(kp, "short_conv") / (hbm * 1e9),
                    "branch_norm_sum_prefill_frac_of_hbm": Lp * T * W * (2.0 + 2 + 4) / us(kp, "branch_norm_sum") / (hbm * 1e9),
                    "retention_out_gate_prefill_frac_of_hbm": Lp * T * H * VDIM * (4.0 + 2 + 2) / us(kp, "retention_out_gate") / (hbm * 1e9),
                    "ssm_thin_products_prefill_us": (us(kp, "ssm_x_proj") + us(kp, "ssm_dt_proj")) * 1e6,
                }
            elif cfgj["architecture"] == "Mulenex":
                att = [ly for ly in cfgj["layers"] if ly["type"] == "attention"]
                rec = [ly for ly in cfgj["layers"] if ly["type"] == "mlstm"]
                G = att[0]["mixer"]["kv_heads"]
                keys = sum(p + 1 for p in range(prompt)) * batch
                att_flops = 2.0 * len(att) * H * keys * (DIM + VDIM)
                scan_flops = 2.0 * 3 * len(rec) * T * H * DIM * (VDIM + 1)
                n_in = len(att) * (H * DIM + G * DIM + G * VDIM + 8) + len(rec) * (2 * H * DIM + 2 * H * VDIM)
                k_out = len(cfgj["layers"]) * H * VDIM
                proj_flops = 2.0 * T * W * (n_in + k_out)
                state_bytes = 2.0 * len(rec) * batch * H * DIM * (VDIM + 1) * 4
                dkeys = batch * (prompt + 1)
                calls = 2 * len(cfgj["layers"]) + 1      # one boundary per sublayer, the last write-back alone
                moes = sum(1 for ly in cfgj["layers"] if ly["mlp"] and ly["mlp"]["kind"] == "moe")
                r["roofline"] = {
                    "attention_prefill_frac_of_bf16_peak": att_flops / us(kp, "attention") / (tf * 1e12),
                    "mlstm_scan_prefill_tflops": scan_flops / us(kp, "mlstm_scan") / 1e12,
                    "projections_prefill_frac_of_bf16_peak": proj_flops / (us(kp, "proj_in") + us(kp, "proj_out")) / (tf * 1e12),
                    "mlstm_scan_decode_frac_of_hbm": state_bytes / us(kd, "mlstm_scan") / (hbm * 1e9),
                    "attention_decode_frac_of_hbm": len(att) * dkeys * G * (DIM + VDIM) * 2.0 / us(kd, "attention") / (hbm * 1e9),
                    "projections_decode_frac_of_hbm": 2.0 * W * (n_in + k_out) / (us(kd, "proj_in") + us(kd, "proj_out")) / (hbm * 1e9),
                    # boundary: reads and writes the fp32 residual, reads a bf16 sublayer output, writes a bf16 row
                    "residual_norm_prefill_frac_of_hbm": calls * T * W * (8.0 + 2 + 2) / us(kp, "residual_norm") / (hbm * 1e9),
                    "moe_experts_prefill_frac_of_bf16_peak": 2.0 * moes * T * z["top"] * 3 * W * z["eff"] / (us(kp, "moe_up") + us(kp, "moe_down")) / (tf * 1e12),
                    "dense_ff_prefill_frac_of_bf16_peak": 2.0 * T * 2 * W * z["ff"] / (us(kp, "ff_up") + us(kp, "ff_down")) / (tf * 1e12),
                    # gate chain, out gate: the small kernels around the scan, as time beside the scan's
                    "mlstm_gates_prefill_us": us(kp, "mlstm_gates") * 1e6 + us(kp, "mlstm_gate_proj") * 1e6,
                    "mlstm_out_gate_prefill_frac_of_hbm": len(rec) * T * H * ((VDIM + 1) * 4.0 + VDIM * 2 + VDIM * 2) / us(kp, "mlstm_out_gate") / (hbm * 1e9),
                }
            else:
                L = len(cfgj["layers"])
                lf = cfgj["layers"][0]["mixer"]["left"]
                G, ns = lf["kv_heads"], cfgj["streams"]
                keys = sum(min(p + 1, z["window"]) + min(lf["mask"]["keep_first"], max(0, p + 1 - z["window"])) for p in range(prompt)) * batch
                att_flops = 2.0 * L * H * keys * (DIM + VDIM)
                scan_flops = 2.0 * 3 * L * T * H * DIM * VDIM
                n_in = L * (H * DIM + G * DIM + G * VDIM + H * VDIM + 2 * H * DIM + 2 * H * VDIM)
                k_out = L * 2 * H * VDIM
                proj_flops = 2.0 * T * W * (n_in + k_out)
                state_bytes = 2.0 * L * batch * H * DIM * VDIM * 4
                dkeys = batch * (min(prompt + 1, z["window"]) + min(lf["mask"]["keep_first"], max(0, prompt + 1 - z["window"])))
                calls = 2 * L + 1      # one boundary per sublayer, the last write-back alone (the head's norm touches `batch` rows)
                r["roofline"] = {
                    "window_attention_prefill_frac_of_bf16_peak": att_flops / us(kp, "window_attention") / (tf * 1e12),
                    "lightning_scan_prefill_tflops": scan_flops / us(kp, "lightning_scan") / 1e12,
                    "projections_prefill_frac_of_bf16_peak": proj_flops / (us(kp, "proj_in") + us(kp, "proj_out")) / (tf * 1e12),
                    "lightning_scan_decode_frac_of_hbm": state_bytes / us(kd, "lightning_scan") / (hbm * 1e9),
                    "window_attention_decode_frac_of_hbm": L * dkeys * G * (DIM + VDIM) * 2.0 / us(kd, "window_attention") / (hbm * 1e9),
                    "projections_decode_frac_of_hbm": 2.0 * W * (n_in + k_out) / (us(kd, "proj_in") + us(kd, "proj_out")) / (hbm * 1e9),
                    # stream boundary: reads and writes `ns` fp32 streams, reads a bf16 sublayer output, writes a bf16 row
                    "stream_norm_prefill_frac_of_hbm": calls * T * W * (8.0 * ns + 2 + 2) / us(kp, "stream_norm") / (hbm * 1e9),
                    "moe_experts_prefill_frac_of_bf16_peak": 2.0 * L * T * z["top"] * 3 * W * z["eff"] / (us(kp, "moe_up") + us(kp, "moe_down")) / (tf * 1e12),
                }
    return r


def bench_size(design, name, z, batch, prompt, decode_steps, warmup, peaks):
    import torch
    from .engine import Engine, default_config
    hbm, tf, _ = peaks
    buf = torch.zeros(160 << 20, dtype=torch.int16, device="cuda")   # 320 MB > 126 MB of L2
    lim = dict(manual_step=1, enable_prefix_caching=0, max_num_seqs=batch, max_batched_tokens=batch * prompt,
               max_model_len=prompt + warmup + decode_steps + 64, record_steps=4, seed=1)
    lim["num_kv_blocks"] = batch * ((lim["max_model_len"] + 15) // 16)
    res = {"size": dict(z, batch=batch, prompt=prompt)}
    T = batch * prompt
    if design == "nagilix":
        res["nagilix"] = run_design(nagilix_config(z), lim, z, batch, prompt, decode_steps, warmup, peaks, torch, buf)
        res["zinavik"] = run_design(zinavik_config(z), lim, z, batch, prompt, decode_steps, warmup, peaks, torch, buf)
        del buf
        return res
    if design == "mulenex":
        res["mulenex"] = run_design(mulenex_config(z), lim, z, batch, prompt, decode_steps, warmup, peaks, torch, buf)
        res["zinavik"] = run_design(zinavik_config(z), lim, z, batch, prompt, decode_steps, warmup, peaks, torch, buf)
        del buf
        return res
    if design == "zinavik":
        res["zinavik"] = run_design(zinavik_config(z), lim, z, batch, prompt, decode_steps, warmup, peaks, torch, buf)
        res["nomanex"] = run_design(nomanex_config(z), lim, z, batch, prompt, decode_steps, warmup, peaks, torch, buf)
        del buf
        return res
    res["nomanex"] = run_design(nomanex_config(z), lim, z, batch, prompt, decode_steps, warmup, peaks, torch, buf)
    # the closest existing model: Llama at equal width, depth, heads x 128 and feed-forward size
    lcfg = default_config(num_layers=4, hidden=z["width"], q_heads=z["heads"], kv_heads=z["heads"] // 4, intermediate=z["ff"],
                          vocab=z["vocab"], **lim)
    with Engine(lcfg) as e:
        r, rids = run_engine(e, torch, buf, z["vocab"], batch, prompt, decode_steps, warmup)
        cls, tot = e.profile_range(1, 1, batch)            # the last decode step
        r["kernels_decode_us"] = {k: round(v["us"], 1) for k, v in cls.items() if v["launches"]}
        for q in rids:
            e.feed_close(q)
        rng = np.random.default_rng(1)
        rids = [e.feed_open() for _ in range(batch)]
        e.feed_step([(q, rng.integers(0, z["vocab"], size=prompt).tolist(), [prompt - 1]) for q in rids])
        cls, tot = e.profile_range(1, batch + 1, 1 << 30)
        r["kernels_prefill_us"] = {k: round(v["us"], 1) for k, v in cls.items() if v["launches"]}
        Hq, Wd, I = z["heads"], z["width"], z["ff"]
        keys = sum(p + 1 for p in range(prompt)) * batch
        att_flops = 4.0 * 4 * Hq * 128 * keys
        pj = [k for k in ("gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down") if k in r["kernels_prefill_us"]]
        proj_flops = 2.0 * T * 4 * (Wd * (Hq + Hq // 2) * 128 + Wd * Hq * 128 + 3 * Wd * I)
        dk = r["kernels_decode_us"]
        r["roofline"] = {
            "attention_prefill_frac_of_bf16_peak": att_flops / (r["kernels_prefill_us"]["attn_prefill"] * 1e-6) / (tf * 1e12),
            "projections_prefill_frac_of_bf16_peak": proj_flops / (sum(r["kernels_prefill_us"][k] for k in pj) * 1e-6) / (tf * 1e12),
            "attention_decode_frac_of_hbm": 4.0 * batch * (prompt + warmup + decode_steps) * (Hq // 4) * 128 * 2 * 2 / (dk["attn_decode"] * 1e-6) / (hbm * 1e9),
            "projections_decode_frac_of_hbm": 2.0 * 4 * (Wd * (Hq + Hq // 2) * 128 + Wd * Hq * 128 + 3 * Wd * I) /
                                              (sum(dk[k] for k in ("gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down") if k in dk) * 1e-6) / (hbm * 1e9),
        }
        res["llama"] = r
    del buf
    return res


def _n_in(ly, W):
    mx = ly["mixer"]
    if ly["type"] == "gla":
        n = 2 * mx["heads"] * mx["dim"] + 2 * mx["heads"] * mx["vdim"] + 16
    else:
        n = mx["heads"] * (mx["dim"] + mx["rot_dim"]) + mx["kv_rank"] + mx["rot_dim"] + mx["heads"] * mx["vdim"]
    return n + (2 * ly["mlp"]["ff"] if ly["mlp"]["kind"] == "dense" else 0)


def _k_out(ly):
    return ly["mixer"]["heads"] * ly["mixer"]["vdim"] + (ly["mlp"]["ff"] if ly["mlp"]["kind"] == "dense" else 0)


def run(design, peaks, sizes=None, batch=8, prompt=512, decode_steps=8, warmup=3):
    if design not in ("nomanex", "zinavik", "mulenex", "nagilix"):
        raise SystemExit("unknown design %r (known: nomanex, zinavik, mulenex, nagilix)" % design)
    out = {"design": design, "dtype": "bf16", "data": "synthetic (seeded random weights and tokens)", "peaks": dict(hbm_gbs=peaks[0], bf16_tflops=peaks[1], source=peaks[2]),
           "timing": "CUDA events around the engine step, median of the timed steps, %d warm-up steps, 320 MB written between steps" % warmup,
           "sizes": {}}
    for name in sizes or list(SIZES):
        out["sizes"][name] = bench_size(design, name, SIZES[name], batch, prompt, decode_steps, warmup, peaks)
    return out
