"""A slow float64 restatement of the Nagilix design, one token at a time, one function per mechanism.

It shares nothing with the CUDA path: plain numpy on the tensors of a checkpoint, every sequence advanced token by
token through explicit per-layer state objects (lists of past keys, carried convolution inputs, recurrent matrices).

Notation.  A model has `streams` copies x_1..x_n of the residual (or one plain residual).  A sublayer f with stream
weights (in, out, mix), norm number g and gate (R, b) does

    u = sum_s in[s] x_s,   h = g * u / sqrt(mean(u^2) + eps),   y = f(h) * sigmoid(R h + b),
    x_j <- sum_s mix[s, j] x_s + out[j] y.

Mixers: `parallel` = 1/2 (w_l * N(left(h)) + w_r * N(right(h))) with N the unit-RMS norm over the width; `mamba1` = the
selective scan.  Feed-forward: routed clamped experts among which the last `identity` router outputs are identity maps.
"""
from __future__ import annotations

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def unit_rms(v, eps):
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    v = np.asarray(v, dtype=np.float64)
    return v / np.sqrt((v * v).mean(axis=-1, keepdims=True) + eps)


def rotate_half(v, p, rot):
    """Rotate the first rot['dims'] entries of every row of v [heads, dim] by position p; entry i pairs with i + dims/2."""
    if not rot or not rot.get("dims"):
        return v
    n = rot["dims"]
    half = n // 2
    ang = p * rot["base"] ** (-2.0 * np.arange(half) / n)
    c, s = np.cos(ang), np.sin(ang)
    out = np.array(v, dtype=np.float64, copy=True)
    a, b = v[..., :half], v[..., half:n]
    out[..., :half] = a * c - b * s
    out[..., half:n] = b * c + a * s
    return out


def chunk_visible(i, j, size):
    """Query position i sees key position j: not later, and in the same chunk of `size` positions (None: plain causal)."""
    return j <= i and (size is None or i // size == j // size)


def sink_softmax(scores, sink):
    """Weights of the given scores when the denominator also holds exp(sink)."""
    m = max(np.max(scores), sink)
    e = np.exp(scores - m)
    return e / (e.sum() + np.exp(sink - m))


class CarriedConv:
    """Causal convolution over time per channel: y_t = b + sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""

    def __init__(self, w, b=None):
        self.w = np.asarray(w, dtype=np.float64)
        self.b = b
        self.past = [np.zeros(self.w.shape[0]) for _ in range(self.w.shape[1] - 1)]

    def step(self, u):
        seq = self.past + [u]
        y = sum(self.w[:, j] * seq[j] for j in range(self.w.shape[1]))
        self.past = seq[1:]
        return y if self.b is None else y + self.b


class LeftBranch:
    """Softmax attention on convolved, whole-row-normed, rotated queries and keys; values are the convolved keys."""

    def __init__(self, P, mx, eps):
        self.P, self.mx, self.eps = P, mx, eps
        self.H, self.G, self.D = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"]
        taps = mx.get("conv") or 1
        self.cq = CarriedConv(P["q.conv"]) if taps > 1 else None
        self.ck = CarriedConv(P["k.conv"]) if taps > 1 else None
        self.keys, self.values = [], []

    def step(self, h):
        P, mx, H, G, D = self.P, self.mx, self.H, self.G, self.D
        p = len(self.keys)
        q, k = P["q"] @ h, P["k"] @ h
        if self.cq:
            q, k = self.cq.step(q), self.ck.step(k)
        self.values.append(k.reshape(G, D))
        q = (unit_rms(q, self.eps) * P["q.norm"]).reshape(H, D)
        k = (unit_rms(k, self.eps) * P["k.norm"]).reshape(G, D)
        q, k = rotate_half(q, p, mx.get("rot")), rotate_half(k, p, mx.get("rot"))
        self.keys.append(k)
        size = (mx.get("mask") or {}).get("size")
        seen = [j for j in range(p + 1) if chunk_visible(p, j, size)]
        out = np.zeros((H, D))
        for hd in range(H):
            g = hd // (H // G)
            s = np.array([q[hd] @ self.keys[j][g] for j in seen]) * mx["scale"] * P["temp"][hd]
            w = sink_softmax(s, P["sink"][hd])
            out[hd] = sum(wj * self.values[j][g] for wj, j in zip(w, seen))
        return P["o"] @ out.reshape(-1)


class RightBranch:
    """Retention: S <- decay_h S + k v^T, o = S^T q, per-head unit-RMS norm, SiLU gate."""

    def __init__(self, P, mx, eps):
        self.P, self.mx, self.eps = P, mx, eps
        self.S = np.zeros((mx["heads"], mx["dim"], mx["vdim"]))
        self.p = 0

    def step(self, h):
        P, mx = self.P, self.mx
        H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
        q = rotate_half((P["q"] @ h).reshape(H, D), self.p, mx.get("rot"))
        k = rotate_half((P["k"] @ h).reshape(H, D), self.p, mx.get("rot")) * D ** -0.5
        v = (P["v"] @ h).reshape(H, Dv)
        self.p += 1
        o = np.zeros((H, Dv))
        for hd in range(H):
            self.S[hd] = mx["decay"][hd] * self.S[hd] + np.outer(k[hd], v[hd])
            o[hd] = self.S[hd].T @ q[hd]
        o = unit_rms(o, self.eps).reshape(-1)
        return P["o"] @ (o * silu(P["g"] @ h))


class ParallelMixer:
    def __init__(self, P, mx, eps):
        self.P, self.eps = P, eps
        self.left, self.right = LeftBranch(sub(P, "left."), mx["left"], eps), RightBranch(sub(P, "right."), mx["right"], eps)

    def step(self, h):
        a = unit_rms(self.left.step(h), self.eps) * self.P["left.out"]
        b = unit_rms(self.right.step(h), self.eps) * self.P["right.out"]
        return 0.5 * (a + b)


class MambaMixer:
    """Selective scan: S[c, n] <- exp(d_c A[c, n]) S[c, n] + d_c x_c B_n;  y_c = S[c, :] . C + D_c x_c."""

    def __init__(self, P, mx, eps):
        self.P, self.mx = P, mx
        self.conv = CarriedConv(P["conv"], P["conv.b"])
        self.A = -np.exp(P["A_log"])
        self.S = np.zeros((mx["inner"], mx["state"]))

    def step(self, h):
        P, mx = self.P, self.mx
        I, N, R = mx["inner"], mx["state"], mx["dt_rank"]
        xz = P["in"] @ h
        x, z = silu(self.conv.step(xz[:I])), xz[I:]
        low = P["x"] @ x
        d = softplus(P["dt"] @ low[:R] + P["dt.b"])
        B, C = low[R:R + N], low[R + N:]
        self.S = np.exp(d[:, None] * self.A) * self.S + (d * x)[:, None] * B[None, :]
        return P["o"] @ ((self.S @ C + P["D"] * x) * silu(z))


def route(P, h, router):
    """(chosen experts in the order of choice, their weights, the margin of the closest call)."""
    z = P["router"] @ h
    s = np.exp(z - z.max())
    s = s / s.sum()
    rank = s + P["correction"]
    order = sorted(range(len(s)), key=lambda e: (-rank[e], e))
    top = router["top"]
    margin = rank[order[top - 1]] - rank[order[top]] if top < len(s) else np.inf
    return order[:top], [s[e] for e in order[:top]], margin


def clamped_expert(P, h, limit):
    g = np.minimum(P["gate"] @ h, limit)
    u = np.clip(P["up"] @ h, -limit, limit)
    return P["down"] @ (g * sigmoid(1.702 * g) * (u + 1.0))


def moe_ff(P, mlp, h):
    E = mlp["router"]["experts"]
    chosen, weights, _ = route(P, h, mlp["router"])
    y = np.zeros_like(h)
    for e, w in zip(chosen, weights):
        y = y + w * (h if e >= E else clamped_expert(sub(P, "e%d." % e), h, mlp["expert"].get("limit", np.inf)))
    return y


def streams_read(xs, hc):
    if hc is None:
        return xs[0]
    return sum(hc["in"][s] * xs[s] for s in range(len(xs)))


def streams_write(xs, hc, y):
    if hc is None:
        return [xs[0] + y]
    n = len(xs)
    return [sum(hc["mix"][s, j] * xs[s] for s in range(n)) + hc["out"][j] * y for j in range(n)]


def sub(P, prefix):
    return {k[len(prefix):]: v for k, v in P.items() if k.startswith(prefix)}


class NagilixOracle:
    def __init__(self, cfg, W):
        self.cfg = cfg
        self.W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
        self.eps = cfg["norm"]["eps"]
        self.gated = "l0.rg1" in self.W

    def _hc(self, layer, q):
        if not self.cfg.get("streams"):
            return None
        return sub(self.W, "l%d.hc%d." % (layer, q))

    def new_state(self):
        out = []
        for i, L in enumerate(self.cfg["layers"]):
            kind = ParallelMixer if L["type"] == "parallel" else MambaMixer
            out.append([kind(sub(self.W, "l%d.mix." % i), L["mixer"], self.eps), 0])
        return out

    def _sublayer(self, xs, li, q, f):
        W = self.W
        hc = self._hc(li, q)
        h = unit_rms(streams_read(xs, hc), self.eps) * float(W["l%d.norm%d" % (li, q)])
        y = f(h)
        if self.gated:
            y = y * sigmoid(W["l%d.rg%d" % (li, q)] @ h + W["l%d.rg%d.b" % (li, q)])
        return streams_write(xs, hc, y)

    def step(self, state, token, layers_out=None, margins_out=None):
        """Advance one sequence by one token; returns its logits."""
        cfg, W = self.cfg, self.W
        p = state[0][1]
        x0 = W["embed"][token] + W["pos"][p]
        xs = [x0.copy() for _ in range(cfg.get("streams") or 1)]
        for li, st in enumerate(state):
            L = cfg["layers"][li]
            st[1] += 1
            xs = self._sublayer(xs, li, 1, st[0].step)
            if L.get("mlp"):
                P = sub(W, "l%d.mlp." % li)

                def ff(h, P=P, L=L):
                    if margins_out is not None:
                        margins_out.append(route(P, h, L["mlp"]["router"])[2])
                    return moe_ff(P, L["mlp"], h)
                xs = self._sublayer(xs, li, 2, ff)
            if layers_out is not None:
                layers_out.append(sum(xs))
        return (W["head"] @ (unit_rms(sum(xs), self.eps) * float(W["final.norm"]))) * cfg.get("logit_scale", 1.0)

    def forward(self, tokens, return_layers=False):
        """Logits of every position [T, vocab]; with return_layers also the summed streams after every layer."""
        state = self.new_state()
        logits, per_tok = [], []
        for t in tokens:
            lo = []
            logits.append(self.step(state, int(t), lo))
            per_tok.append(lo)
        out = np.stack(logits)
        if return_layers:
            return out, np.stack([[per_tok[t][r] for t in range(len(tokens))] for r in range(len(self.cfg["layers"]))])
        return out

    def routing_margins(self, tokens):
        """Per position, the smallest router margin over all layers (inf for a model without routing decisions)."""
        state = self.new_state()
        out = []
        for t in tokens:
            m = []
            self.step(state, int(t), None, m)
            out.append(min(m) if m else float("inf"))
        return np.array(out)

    def generate(self, prompt, n):
        """Greedy continuation: (tokens, smallest top-1 / top-2 margin met on the way)."""
        state = self.new_state()
        lg = None
        for t in prompt:
            lg = self.step(state, int(t))
        out, margin = [], float("inf")
        for _ in range(n):
            top = np.sort(lg)[-2:]
            margin = min(margin, top[1] - top[0])
            nxt = int(np.argmax(lg))
            out.append(nxt)
            lg = self.step(state, nxt)
        return out, margin
