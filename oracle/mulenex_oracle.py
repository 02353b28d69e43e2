"""TEST INFRASTRUCTURE — plain, slow restatement of the Mulenex decoder, one function per mechanism.

Mulenex is a decoder on one residual stream with a norm on both sides of every sublayer ("sandwich"):

    x <- x + N_1b(mixer(N_1(x))),   x <- x + N_2b(ff(N_2(x))),   N(u) = u / sqrt(mean(u^2) + eps) * (1 + w)

The input is the token's embedding row plus a sinusoidal position row.  A layer's mixer is either a matrix-memory
recurrence with exponential gating (the mLSTM cell of xLSTM: a per-head matrix C, a normaliser vector n and a running
log-scale m) or softmax attention with grouped key/value heads, a weighted RMS norm of every query and key head, no
rotation, a query gain that grows with the logarithm of the position in steps, tanh-capped scores, values blended with
the values of the first blending layer, and one sigmoid output gate per head.  The feed-forward is a squared-ReLU layer
with biases, or a mixture of SiLU-gated experts chosen by the largest biased router logits and weighted by the softmax
over the chosen logits only, plus a shared expert behind a one-number sigmoid gate; a layer may have none.

Everything here runs token by token in float64 on the CPU and keeps its caches in plain arrays.  It shares no code with
the CUDA path (kubeai_b200/csrc/mulenex.cu and the kernels it launches); tests compare the engine against it.
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return np.minimum(z, 0.0) - np.log1p(np.exp(-np.abs(z)))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight is the offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


def soft_cap(z, cap):
    """cap * tanh(z / cap): the identity near zero, never beyond +-cap."""
    return cap * np.tanh(z / cap)


# ---------------------------------------------------------------- input
def position_row(pos, width, base=10000.0):
    """Column c belongs to the pair i = c // 2 with angle pos * base^(-2i/width): even columns carry its sine, odd its cosine."""
    row = np.zeros(width)
    for c in range(width):
        ang = pos * base ** (-2.0 * (c // 2) / width)
        row[c] = math.sin(ang) if c % 2 == 0 else math.cos(ang)
    return row


# ---------------------------------------------------------------- mixer: matrix memory with exponential gating
class MatrixMemory:
    """Per head: C [dim, vdim], n [dim], m (log of the scale the stored C and n are divided by; 0 at the start)."""

    def __init__(self, P, mx, eps):
        self.P, self.mx, self.eps = P, mx, eps
        H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
        self.C = np.zeros((H, D, Dv))
        self.n = np.zeros((H, D))
        self.m = np.zeros(H)

    def gates(self, h):
        """log input gate and log forget gate of every head, both through a tanh cap on the pre-activation"""
        P, cap = self.P, self.mx["gate_cap"]
        li = soft_cap(P["i"] @ h + P["i.b"], cap)
        lf = log_sigmoid(soft_cap(P["f"] @ h + P["f.b"], cap))
        return li, lf

    def step(self, h):
        mx, P = self.mx, self.P
        H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
        q = (P["q"] @ h).reshape(H, D) * D ** -0.5
        k = (P["k"] @ h).reshape(H, D)
        v = (P["v"] @ h).reshape(H, Dv)
        li, lf = self.gates(h)
        out = np.zeros((H, Dv))
        for a in range(H):
            m_new = max(lf[a] + self.m[a], li[a])
            keep, take = math.exp(lf[a] + self.m[a] - m_new), math.exp(li[a] - m_new)
            self.C[a] = keep * self.C[a] + take * np.outer(k[a], v[a])
            self.n[a] = keep * self.n[a] + take * k[a]
            self.m[a] = m_new
            den = max(abs(self.n[a] @ q[a]), math.exp(-m_new)) + 1e-6
            out[a] = (self.C[a].T @ q[a]) / den
        y = unit_rms(out, self.eps).reshape(-1) * P["norm"] * sigmoid(P["g"] @ h)
        return P["o"] @ y


# ---------------------------------------------------------------- mixer: softmax attention
def query_gain(pos, q_temp):
    """1 + coef * ln(floor((pos + 1) / every) + 1): constant over runs of `every` positions, 1 for the first every - 1."""
    if not q_temp:
        return 1.0
    return 1.0 + q_temp["coef"] * math.log((pos + 1) // q_temp["every"] + 1)


class Attention:
    def __init__(self, P, mx, eps, blend_source):
        """blend_source: None (no value blending, or this is the first blending layer), else the Attention whose raw
        values of the same token are blended in."""
        self.P, self.mx, self.eps, self.src = P, mx, eps, blend_source
        self.keys, self.values = [], []     # per position: [kv_heads, dim], [kv_heads, vdim]
        self.raw_value = None               # this token's values before any blending

    def step(self, h):
        mx, P = self.mx, self.P
        H, G, D, Dv = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
        pos = len(self.keys)
        q = unit_rms((P["q"] @ h).reshape(H, D), self.eps) * P["q.norm"] * query_gain(pos, mx.get("q_temp"))
        k = unit_rms((P["k"] @ h).reshape(G, D), self.eps) * P["k.norm"]
        v = (P["v"] @ h).reshape(G, Dv)
        self.raw_value = v
        if self.src is not None:
            lam = float(P["vmix"])
            v = (1.0 - lam) * v + lam * self.src.raw_value
        self.keys.append(k)
        self.values.append(v)
        K, V = np.stack(self.keys), np.stack(self.values)       # [pos + 1, G, .]
        gate = sigmoid(P["g"] @ h)                              # one number per head
        heads = []
        for a in range(H):
            g = a // (H // G)
            s = (K[:, g] @ q[a]) * mx["scale"]
            if mx.get("softcap"):
                s = soft_cap(s, mx["softcap"])
            w = np.exp(s - s.max())
            w /= w.sum()
            heads.append((w @ V[:, g]) * gate[a])
        return P["o"] @ np.concatenate(heads)


# ---------------------------------------------------------------- feed-forward
def dense_ff(P, h):
    """squared ReLU between two biased projections"""
    return P["down"] @ np.maximum(P["up"] @ h + P["up.b"], 0.0) ** 2 + P["down.b"]


def gated_expert(P, prefix, h):
    return P[prefix + "down"] @ (silu(P[prefix + "gate"] @ h) * (P[prefix + "up"] @ h))


def route(logits, top):
    """The `top` largest logits (ties to the lower index) and the softmax over just those."""
    order = sorted(range(len(logits)), key=lambda e: (-logits[e], e))[:top]
    z = np.array([logits[e] for e in order])
    w = np.exp(z - z.max())
    return order, w / w.sum()


def moe_ff(P, mlp, h):
    logits = P["router"] @ h + P["router.b"]
    chosen, weights = route(logits, mlp["router"]["top"])
    y = sum(w * gated_expert(P, "e%d." % e, h) for e, w in zip(chosen, weights))
    if mlp.get("shared"):
        y = y + sigmoid((P["shared.sg"] @ h).item()) * gated_expert(P, "shared.", h)
    return y


def routing_margin(P, mlp, h):
    """Gap between the last chosen and the first rejected router logit (inf when every expert is chosen)."""
    z = np.sort(P["router"] @ h + P["router.b"])[::-1]
    top = mlp["router"]["top"]
    return math.inf if top >= len(z) else float(z[top - 1] - z[top])


# ---------------------------------------------------------------- the model
class MulenexOracle:
    def __init__(self, cfg, weights):
        self.cfg = cfg
        self.W = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
        self.eps = cfg["norm"]["eps"]
        self.mlp_weights = [self.sub("l%d.mlp." % i) for i in range(len(cfg["layers"]))]

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.W.items() if k.startswith(prefix)}

    def new_mixers(self):
        mixers, first_blend = [], None
        for i, ly in enumerate(self.cfg["layers"]):
            P = self.sub("l%d.mix." % i)
            if ly["type"] == "mlstm":
                mixers.append(MatrixMemory(P, ly["mixer"], self.eps))
            elif ly["type"] == "attention":
                blends = bool(ly["mixer"].get("v_mix"))
                a = Attention(P, ly["mixer"], self.eps, first_blend if blends else None)
                if blends and first_blend is None:
                    first_blend = a
                mixers.append(a)
            else:
                raise ValueError(ly["type"])
        return mixers

    def new_state(self):
        return dict(mixers=self.new_mixers(), pos=0)

    def step(self, state, tok, layers=None, margin=None):
        """One token through every layer; returns its logits.  `layers` collects the residual after every layer,
        `margin` (a one-element list) the smallest routing margin met."""
        W, cfg, eps = self.W, self.cfg, self.eps
        x = W["embed"][tok] + position_row(state["pos"], cfg["width"])
        state["pos"] += 1
        for i, ly in enumerate(cfg["layers"]):
            p = "l%d." % i
            y = state["mixers"][i].step(norm_one_plus(x, W[p + "norm1"], eps))
            x = x + norm_one_plus(y, W[p + "norm1b"], eps)
            mlp = ly.get("mlp")
            if mlp:
                h = norm_one_plus(x, W[p + "norm2"], eps)
                P = self.mlp_weights[i]
                if mlp["kind"] == "dense":
                    y = dense_ff(P, h)
                else:
                    y = moe_ff(P, mlp, h)
                    if margin is not None:
                        margin[0] = min(margin[0], routing_margin(P, mlp, h))
                x = x + norm_one_plus(y, W[p + "norm2b"], eps)
            if layers is not None:
                layers.append(x.copy())
        return W["head"] @ norm_one_plus(x, W["final.norm"], eps)

    def forward(self, tokens, return_layers=False, return_margins=False):
        """Logits [n, vocab] of every position (optionally the residual after every layer [layers, n, width], or per
        position the smallest routing margin over the layers)."""
        state = self.new_state()
        logits, layers, margins = [], [], []
        for tok in tokens:
            per_layer, margin = [], [math.inf]
            logits.append(self.step(state, int(tok), per_layer, margin))
            layers.append(per_layer)
            margins.append(margin[0])
        out = np.stack(logits)
        if return_layers:
            return out, np.stack(layers).transpose(1, 0, 2)
        if return_margins:
            return out, np.array(margins)
        return out

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

    def routing_margins(self, tokens):
        return self.forward(tokens, return_margins=True)[1]
