"""Plain, slow float64 restatement of the Latanex decoder (numpy only; one function per mechanism).

The design: x0 = embed[token] * s_e.  Every sublayer sits between two element-wise norms, x <- x + N_b(f(N_a(x))), where
N(x) = tanh(a x) * w + b has a scalar a and vectors w, b and needs no statistic of the row.  Mixers:
  * windowed grouped-query attention with biased q / k / v projections, a unit-RMS norm over the WHOLE q (and k) projection
    with a gain per entry, no rotation, tanh-capped scores, a learned per-head sink in the softmax denominator and values
    blended with the values the first blending layer produced for the same token;
  * a gated delta rule: short causal convolutions + silu on q, k, v, unit-length q and k, a scalar decay and a scalar write
    strength per head, S <- g S; S <- S + k (beta (v - S^T k))^T; o = S^T q, per-head RMS norm and a silu gate.
Feed-forwards: silu-gated unit, or a mixture of clamped experts chosen by a sigmoid router with choice corrections and a
restriction to the best groups of neighbouring experts, plus a shared expert.  Logits = head N(x) * s_l.
Notation: T tokens, W width, H / G query / key-value heads, D / Dv per-head key / value size.  Nothing here is shared with
the CUDA path.
"""
import math

import numpy as np

F = np.float64


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, F)))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    z = np.asarray(z, F)
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def tanh_norm(x, p, name):
    """N(x) = tanh(alpha x) * w + b with the tensors name, name.alpha, name.b of p."""
    return np.tanh(float(p[name + ".alpha"]) * np.asarray(x, F)) * np.asarray(p[name], F) + np.asarray(p[name + ".b"], F)


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, F)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


# ------------------------------------------------------------------ attention
def window_visible(i, j, size):
    """Position i sees j: 0 <= i - j < size (size None or <= 0: every j <= i)."""
    return j <= i and (not size or size <= 0 or i - j < size)


def attention_qkv(h, p, m, eps):
    """-> q [T, H, D] and k [T, G, D] (each normed over its whole projection, then split into heads), v [T, G, Dv] raw."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit(h @ p["q"].T + p["q.b"], eps) * p["q.norm"]
    k = rms_unit(h @ p["k"].T + p["k.b"], eps) * p["k.norm"]
    v = h @ p["v"].T + p["v.b"]
    return q.reshape(T, H, D), k.reshape(T, G, D), v.reshape(T, G, Dv)


def blend_values(v, v_first, lam):
    """v <- (1 - lam) v + lam v_first; the first blending layer passes v_first = None and keeps its own values."""
    return v if v_first is None else (1.0 - lam) * v + lam * v_first


def capped(s, cap):
    return s if not cap or cap <= 0 else cap * np.tanh(s / cap)


def sink_softmax(s, sink):
    """Weights of the scores s when exp(sink) joins the denominator (sink None: plain softmax)."""
    mx = s.max() if sink is None else max(s.max(), sink)
    e = np.exp(s - mx)
    return e / (e.sum() + (0.0 if sink is None else math.exp(sink - mx)))


def attention_mixer(h, p, m, eps, pos=None, past=None, v_first=None):
    """h [T, W] at positions pos -> ([T, W], (keys, blended values, positions) including the past, this call's raw-or-blended
    values [T, G, Dv]).  v_first [T, G, Dv]: the first blending layer's values of the same tokens, None in that layer itself
    or when the layer does not blend."""
    T = h.shape[0]
    H, G = m["heads"], m["kv_heads"]
    pos = np.arange(T) if pos is None else np.asarray(pos)
    q, k, v = attention_qkv(h, p, m, eps)
    if m.get("v_mix"):
        v = blend_values(v, v_first, float(p["vmix"]))
    v_new = v
    if past is not None:
        k, v, kpos = np.concatenate([past[0], k]), np.concatenate([past[1], v]), np.concatenate([past[2], pos])
    else:
        kpos = pos
    size = (m.get("mask") or {}).get("size")
    use_sink = m.get("sink", True)  # the design always has it; tests switch it off to show that it matters
    out = np.zeros((T, H, v.shape[-1]), F)
    for t in range(T):
        see = np.array([window_visible(int(pos[t]), int(j), size) for j in kpos])
        for hh in range(H):
            g = hh // (H // G)
            s = capped((k[see, g] @ q[t, hh]) * m["scale"], m.get("softcap"))
            out[t, hh] = sink_softmax(s, float(p["sink"][hh]) if use_sink else None) @ v[see, g]
    return out.reshape(T, -1) @ p["o"].T, (k, v, kpos), v_new


# ------------------------------------------------------------------ gated delta rule
def short_conv(x, w, tail=None):
    """Causal per-channel convolution over time.  x [T, C], w [C, taps] (last column multiplies the current token), tail
    [taps-1, C] the inputs before x (zeros at the start of a sequence) -> (y [T, C], new tail)."""
    taps = w.shape[1]
    tail = np.zeros((taps - 1, x.shape[1]), F) if tail is None else tail
    ext = np.concatenate([tail, np.asarray(x, F)])
    y = np.zeros_like(np.asarray(x, F))
    for j in range(taps):
        y += ext[j:j + x.shape[0]] * w[:, j]
    return y, ext[ext.shape[0] - (taps - 1):]


def unit_vector(x):
    x = np.asarray(x, F)
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)


def delta_step(S, q, k, v, g, beta):
    """One token of one head.  S [D, Dv]: decay, write the error of the prediction S^T k, read with q."""
    S = g * S
    u = beta * (v - S.T @ k)
    S = S + np.outer(k, u)
    return S, S.T @ q


def delta_mixer(h, p, m, eps, state=None):
    """h [T, W] -> ([T, W], state).  state = dict(S [H, D, Dv], q / k / v convolution tails); None = start of a sequence."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    st = dict(S=np.zeros((H, D, Dv), F), q=None, k=None, v=None) if state is None else dict(state)
    q, st["q"] = short_conv(h @ p["q"].T, p["q.conv"], st["q"])
    k, st["k"] = short_conv(h @ p["k"].T, p["k.conv"], st["k"])
    v, st["v"] = short_conv(h @ p["v"].T, p["v.conv"], st["v"])
    q = unit_vector(silu(q).reshape(T, G, D)) / math.sqrt(D)
    k = unit_vector(silu(k).reshape(T, G, D))
    v = silu(v).reshape(T, H, Dv)
    beta = sigmoid(h @ p["b"].T)                                                    # [T, H]
    g = np.exp(-np.exp(np.asarray(p["A_log"], F)) * softplus(h @ p["a"].T + p["dt_bias"]))  # [T, H]
    S = st["S"].copy()
    o = np.zeros((T, H, Dv), F)
    for t in range(T):
        for hh in range(H):
            kv = hh // (H // G)
            S[hh], o[t, hh] = delta_step(S[hh], q[t, kv], k[t, kv], v[t, hh], g[t, hh], beta[t, hh])
    st["S"] = S
    gate = silu(h @ p["g"].T).reshape(T, H, Dv)
    o = rms_unit(o, eps) * p["norm"] * gate
    return o.reshape(T, -1) @ p["o"].T, st


# ------------------------------------------------------------------ feed-forward
def dense_ff(h, p):
    return (silu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def clamped_expert(h, p, limit):
    g = np.minimum(h @ p["gate"].T, limit)
    u = np.clip(h @ p["up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ p["down"].T


def moe_choice_scores(h, p, r):
    """-> (s, c): s = sigmoid(router h) [T, E]; c = s + correction with every expert outside the kept groups at -inf.
    A group's score is the sum of its two largest corrected scores (of its one score when it holds one expert)."""
    s = sigmoid(np.asarray(h, F) @ p["router"].T)
    c = s + np.asarray(p["correction"], F)
    gr = r.get("groups")
    if gr and gr["count"] > 1 and gr["keep"] < gr["count"]:
        T, E = c.shape
        per = E // gr["count"]
        cg = c.reshape(T, gr["count"], per)
        gs = -np.sort(-cg, axis=-1)[:, :, :2].sum(-1)
        keep = np.argsort(-gs, axis=-1, kind="stable")[:, :gr["keep"]]
        mask = np.full((T, gr["count"]), -np.inf)
        np.put_along_axis(mask, keep, 0.0, -1)
        c = (cg + mask[:, :, None]).reshape(T, E)
    return s, c


def moe_route(h, p, r):
    """-> (chosen experts [T, top], weights [T, top]): weights = uncorrected scores of the chosen / their sum * scale."""
    s, c = moe_choice_scores(h, p, r)
    idx = np.argsort(-c, axis=-1, kind="stable")[:, :r["top"]]
    w = np.take_along_axis(s, idx, -1)
    return idx, w / (w.sum(-1, keepdims=True) + 1e-20) * float(r.get("scale", 1.0))


def route_margin(h, p, r):
    """Per token: the smallest gap that decides the choice — between the last chosen and the first left-out expert, and
    between the last kept and the first dropped group."""
    s, c = moe_choice_scores(h, p, r)
    cs = -np.sort(-c, axis=-1)
    top = r["top"]
    m = cs[:, top - 1] - cs[:, top] if cs.shape[1] > top else np.full(len(cs), np.inf)
    m = np.where(np.isfinite(m), m, np.inf)
    gr = r.get("groups")
    if gr and gr["count"] > 1 and gr["keep"] < gr["count"]:
        raw = (s + np.asarray(p["correction"], F)).reshape(len(s), gr["count"], -1)
        gs = -np.sort(-(-np.sort(-raw, axis=-1)[:, :, :2].sum(-1)), axis=-1)
        m = np.minimum(m, gs[:, gr["keep"] - 1] - gs[:, gr["keep"]])
    return m


def moe_ff(h, p, mlp):
    r = mlp["router"]
    idx, wt = moe_route(h, p, r)
    h = np.asarray(h, F)
    out = np.zeros_like(h)
    lim = float(mlp["expert"]["limit"])
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wt[t]):
            out[t] += w * clamped_expert(h[t], p[f"e{e}"], lim)
    if mlp.get("shared"):
        out += clamped_expert(h, p["shared"], float(mlp["shared"]["limit"]))
    return out


# ------------------------------------------------------------------ the model
def split_params(sd, n_layers):
    """Flat {name: array} of a checkpoint -> per-layer dictionaries of float64 arrays (mix / mlp / norms)."""
    g = lambda k: np.asarray(sd[k], F)
    layers = []
    for i in range(n_layers):
        pre = f"l{i}."
        mix, mlp, norms = {}, {}, {}
        for k in sd:
            if not k.startswith(pre):
                continue
            rest = k[len(pre):]
            if rest.startswith("mix."):
                mix[rest[4:]] = g(k)
            elif rest.startswith("mlp."):
                parts = rest[4:].split(".")
                if len(parts) == 2 and (parts[0] == "shared" or (parts[0][0] == "e" and parts[0][1:].isdigit())):
                    mlp.setdefault(parts[0], {})[parts[1]] = g(k)
                else:
                    mlp[rest[4:]] = g(k)
            else:
                norms[rest] = g(k)
        layers.append(dict(mix=mix, mlp=mlp, norms=norms))
    top = {k: g(k) for k in sd if k.startswith("final.")}
    return dict(embed=g("embed"), head=g("head"), top=top, layers=layers)


class LatanexOracle:
    """The decoder over a checkpoint, fed in portions.  A sequence's state: per attention layer its keys, blended values and
    positions; per delta layer the matrices S and the convolution tails."""

    def __init__(self, cfg, sd):
        self.cfg = cfg
        self.P = split_params(sd, len(cfg["layers"]))
        self.eps = float(cfg["norm"]["eps"])

    def new_state(self):
        return dict(pos=0, layer={})

    def forward(self, tokens, state=None, taps=None, margins=None):
        """The next tokens of one sequence -> logits [T, vocab].  taps / margins (lists) receive the stream after every layer
        / every router's decision margins per token."""
        cfg, P, eps = self.cfg, self.P, self.eps
        st = state if state is not None else self.new_state()
        T = len(tokens)
        pos = st["pos"] + np.arange(T)
        x = P["embed"][np.asarray(tokens)] * float(cfg["embedding"]["scale"])
        v_first = None
        for i, (ly, p) in enumerate(zip(cfg["layers"], P["layers"])):
            n = p["norms"]
            h = tanh_norm(x, n, "norm1")
            if ly["type"] == "attention":
                blends = bool(ly["mixer"].get("v_mix"))
                y, st["layer"][i], v_new = attention_mixer(h, p["mix"], ly["mixer"], eps, pos, st["layer"].get(i), v_first if blends else None)
                if blends and v_first is None:
                    v_first = v_new
            elif ly["type"] == "delta":
                y, st["layer"][i] = delta_mixer(h, p["mix"], ly["mixer"], eps, st["layer"].get(i))
            else:
                raise ValueError(ly["type"])
            x = x + tanh_norm(y, n, "norm1b")
            mlp = ly.get("mlp")
            if mlp:
                h = tanh_norm(x, n, "norm2")
                if margins is not None and mlp["kind"] == "moe":
                    margins.append(route_margin(h, p["mlp"], mlp["router"]))
                y = dense_ff(h, p["mlp"]) if mlp["kind"] == "dense" else moe_ff(h, p["mlp"], mlp)
                x = x + tanh_norm(y, n, "norm2b")
            if taps is not None:
                taps.append(x.copy())
        st["pos"] += T
        return (tanh_norm(x, P["top"], "final.norm") @ P["head"].T) * float(cfg.get("logit_scale", 1.0))

    def greedy(self, prompt, n):
        st = self.new_state()
        z = self.forward(prompt, st)[-1]
        out, rows = [], []
        for _ in range(n):
            rows.append(z)
            out.append(int(np.argmax(z)))
            z = self.forward([out[-1]], st)[-1]
        return out, np.stack(rows)


def forward(cfg, sd, tokens, trace=None):
    """Whole sequence from position 0 -> logits [T, vocab]."""
    return LatanexOracle(cfg, sd).forward(tokens, taps=trace)


# ------------------------------------------------------------------ random checkpoints for tests
def random_config(width=80, vocab=150, order=(("attention", "dense"), ("delta", "moe"), ("attention", "moe"), ("attention", None)),
                  heads=6, kv_heads=2, dim=24, vdim=16, window=20, scale=None, softcap=6.0, v_mix=True,
                  delta=None, ff=72, expert_ff=40, experts=6, groups=(3, 2), top=2, route_scale=1.5, limit=1.5,
                  shared_ff=48, shared_limit=2.0, embed_scale=2.0, logit_scale=0.5, eps=1e-5, per_layer=None):
    """A small configuration; `order` lists each layer's (mixer type, feed-forward kind or None); per_layer[i] overrides mixer
    keys of layer i; delta overrides the delta layers' sizes (heads, kv_heads, dim, vdim, conv)."""
    dl = dict(heads=4, kv_heads=2, dim=16, vdim=24, conv=4)
    dl.update(delta or {})
    layers = []
    for i, (mix, kind) in enumerate(order):
        if mix == "attention":
            mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=float(scale if scale is not None else 2.0 / math.sqrt(dim)),
                         v_mix=bool(v_mix))
            if softcap:
                mixer["softcap"] = float(softcap)
            if window:
                mixer["mask"] = dict(size=int(window))
        else:
            mixer = dict(dl)
        mixer.update((per_layer or {}).get(i, {}))
        if kind == "dense":
            mlp = dict(kind="dense", ff=ff)
        elif kind == "moe":
            router = dict(experts=experts, top=top, scale=float(route_scale))
            if groups:
                router["groups"] = dict(count=groups[0], keep=groups[1])
            mlp = dict(kind="moe", expert=dict(ff=expert_ff, limit=float(limit)), router=router)
            if shared_ff:
                mlp["shared"] = dict(ff=shared_ff, limit=float(shared_limit))
        else:
            mlp = None
        layers.append(dict(type=mix, mixer=mixer, mlp=mlp))
    return dict(architecture="Latanex", width=width, vocab=vocab, layers=layers, norm=dict(eps=eps),
                embedding=dict(scale=float(embed_scale)), logit_scale=float(logit_scale))


def random_state_dict(cfg, seed=0):
    from .weights import _rng, _t, to_bf16_f32
    W, V = cfg["width"], cfg["vocab"]
    s = lambda n: 1.0 / math.sqrt(n)
    sd = {"embed": _t(seed, "embed", (V, W), 0.5), "head": _t(seed, "head", (V, W), s(W))}

    def norm(name):
        sd[name] = _t(seed, name, (W,), 0.1, 1.0)
        sd[name + ".b"] = _t(seed, name + "b", (W,), 0.1)
        sd[name + ".alpha"] = to_bf16_f32(np.float32(0.4 + 0.4 * _rng(seed, name + "a").random())).reshape(())

    norm("final.norm")
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}."
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        norm(p + "norm1")
        norm(p + "norm1b")
        if ly["type"] == "attention":
            sd[p + "mix.q"] = _t(seed, p + "q", (H * D, W), s(W))
            sd[p + "mix.k"] = _t(seed, p + "k", (G * D, W), s(W))
            sd[p + "mix.v"] = _t(seed, p + "v", (G * Dv, W), s(W))
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                sd[p + f"mix.{n}.b"] = _t(seed, p + n + "b", (rows,), 0.2)
            sd[p + "mix.q.norm"] = _t(seed, p + "qn", (H * D,), 0.2, 1.0)
            sd[p + "mix.k.norm"] = _t(seed, p + "kn", (G * D,), 0.2, 1.0)
            sd[p + "mix.vmix"] = to_bf16_f32(np.float32(0.2 + 0.5 * _rng(seed, p + "vm").random())).reshape(())
            sd[p + "mix.sink"] = _t(seed, p + "sink", (H,), 1.0)
            sd[p + "mix.o"] = _t(seed, p + "o", (W, H * Dv), s(H * Dv))
        else:
            taps = m["conv"]
            sd[p + "mix.q"] = _t(seed, p + "q", (G * D, W), 2.0 * s(W))
            sd[p + "mix.k"] = _t(seed, p + "k", (G * D, W), 2.0 * s(W))
            sd[p + "mix.v"] = _t(seed, p + "v", (H * Dv, W), 2.0 * s(W))
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                sd[p + f"mix.{n}.conv"] = _t(seed, p + n + "c", (rows, taps), 0.6)
            sd[p + "mix.b"] = _t(seed, p + "b", (H, W), 2.0 * s(W))
            sd[p + "mix.a"] = _t(seed, p + "a", (H, W), 2.0 * s(W))
            sd[p + "mix.A_log"] = _t(seed, p + "A", (H,), 0.5, -1.5)
            sd[p + "mix.dt_bias"] = _t(seed, p + "dt", (H,), 0.5)
            sd[p + "mix.norm"] = _t(seed, p + "hn", (Dv,), 0.1, 1.0)
            sd[p + "mix.g"] = _t(seed, p + "g", (H * Dv, W), 2.0 * s(W))
            sd[p + "mix.o"] = _t(seed, p + "o", (W, H * Dv), s(H * Dv))
        mlp = ly.get("mlp")
        if not mlp:
            continue
        norm(p + "norm2")
        norm(p + "norm2b")

        def unit(pre, Fn):
            sd[pre + "gate"] = _t(seed, pre + "g", (Fn, W), 2.0 * s(W))
            sd[pre + "up"] = _t(seed, pre + "u", (Fn, W), 2.0 * s(W))
            sd[pre + "down"] = _t(seed, pre + "d", (W, Fn), s(Fn))

        if mlp["kind"] == "dense":
            unit(p + "mlp.", mlp["ff"])
        else:
            r = mlp["router"]
            E = r["experts"]
            sd[p + "mlp.router"] = _t(seed, p + "router", (E, W), 3.0 * s(W))
            # choice corrections on a shuffled grid: no two experts tie by their corrections alone
            sd[p + "mlp.correction"] = to_bf16_f32((_rng(seed, p + "corr").permutation(E) - (E - 1) / 2.0) * 0.0625)
            for e in range(E):
                unit(p + f"mlp.e{e}.", mlp["expert"]["ff"])
            if mlp.get("shared"):
                unit(p + "mlp.shared.", mlp["shared"]["ff"])
    return sd
