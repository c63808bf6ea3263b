"""Plain, slow float64 restatement of the Funudra decoder (numpy only; one function per mechanism).

The design: x0 = rmsnorm(embed[token]) * g_e.  Every layer reads the stream through two RMS norms and adds both sublayers'
outputs in one step: x <- x + mixer(N1(x)) + ff(N2(x)) (the feed-forward may be absent).  Mixers:
  * "mamba2": one input projection laid out [z | x | B | C | dt]; x, B, C pass a short causal convolution (with bias) and
    silu; per head S <- exp(-exp(A) dt) S + dt B x^T with dt = softplus(dt + dt_bias), y = S^T C + D x; y * silu(z) is
    RMS-normed in equal parts of the concatenated heads and projected out;
  * "parallel": two mixers beside each other on the same input, summed with two configured weights.
      left:  grouped-query softmax attention whose biased q / k / v projections pass a short causal convolution (no bias,
             no activation) before the first `dims` entries of every q / k head turn (entry i pairs with i + dims/2,
             angle pos * base^(-2i/dims) / factor); scores are scaled, tanh-capped, causal; the concatenated heads are
             multiplied by sigmoid(W_g h) before the biased output projection;
      right: a matrix memory with exponential gates kept stable by a running maximum m (which starts at 0):
             m' = max(f + m, i);  S' = exp(f + m - m') S + exp(i - m') k v^T;  n' likewise with k alone;
             o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6), q scaled by dim^-1/2; i = cap tanh(z_i / cap),
             f = logsigmoid(cap tanh(z_f / cap)); per-head unit RMS, a gain over all heads' entries, sigmoid(W_g h), W_o.
The feed-forward is W_down relu(W_up h)^2.  A layer may name another layer whose tensors it uses (`weights_of`) while it
keeps a cache and a state of its own.  Logits = embed . rmsnorm(x) * g_f (the embedding table is the output matrix).
Notation: T tokens, W width, H / G query / key-value heads, D / Dv per-head key / value size, N state size.  Nothing here
is shared with the CUDA path.
"""
import copy
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


def logsigmoid(z):
    return -softplus(-np.asarray(z, F))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, F)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * np.asarray(w, F)


def short_conv(u, w, tail=None):
    """Causal convolution per channel: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the sequence's start.
    u [T, C], w [C, taps]; tail [taps - 1, C] = the inputs just before u (None: the sequence starts here).
    -> y [T, C] and the new tail (the last taps - 1 inputs seen so far)."""
    u = np.asarray(u, F)
    C, taps = w.shape
    if tail is None:
        tail = np.zeros((taps - 1, C), F)
    ext = np.concatenate([tail, u], 0)
    y = np.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(taps):
            y[t] += w[:, j] * ext[t + j]
    return y, ext[ext.shape[0] - (taps - 1):].copy()


def rotate_half_layout(x, pos, dims, base, factor=1.0):
    """x [T, heads, D]: entries i and i + dims/2 (i < dims/2) of every head turn by pos * base^(-2i/dims) / factor."""
    x = np.array(x, F)
    half = dims // 2
    if half == 0:
        return x
    f = np.asarray([base ** (-2.0 * i / dims) for i in range(half)], F) / factor
    ang = np.asarray(pos, F)[:, None] * f[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half].copy(), x[..., half:dims].copy()
    x[..., :half] = a * c - b * s
    x[..., half:dims] = b * c + a * s
    return x


def capped(s, cap):
    return cap * np.tanh(s / cap) if cap and cap > 0 else s


def causal_softmax_attention(q, k, v, q_pos, k_pos, scale, cap):
    """q [Tq, H, D], k [Tk, G, D], v [Tk, G, Dv]; query i sees the keys with k_pos <= q_pos[i]. -> [Tq, H, Dv]"""
    Tq, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((Tq, H, v.shape[2]), F)
    for h in range(H):
        g = h // (H // G)
        s = capped((q[:, h] @ k[:, g].T) * scale, cap)
        s = np.where(k_pos[None, :] <= q_pos[:, None], s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(-1, keepdims=True)
        out[:, h] = p @ v[:, g]
    return out


def attention_branch(h, p, m, pos, past=None):
    """The left mixer.  past = dict(k, v, kpos, tails) of the sequence so far. -> output [T, W] and the new past."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    past = past or {}
    tails = dict(past.get("tails") or {})
    proj = {}
    for n in ("q", "k", "v"):
        u = h @ p[n].T + p[n + ".b"]
        if m.get("conv"):
            u, tails[n] = short_conv(u, p[n + ".conv"], tails.get(n))
        proj[n] = u
    q, k, v = proj["q"].reshape(T, H, D), proj["k"].reshape(T, G, D), proj["v"].reshape(T, G, Dv)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        fac = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate_half_layout(q, pos, int(rot["dims"]), float(rot["base"]), fac)
        k = rotate_half_layout(k, pos, int(rot["dims"]), float(rot["base"]), fac)
    if "k" in past:
        k_all, v_all = np.concatenate([past["k"], k], 0), np.concatenate([past["v"], v], 0)
        kpos = np.concatenate([past["kpos"], pos])
    else:
        k_all, v_all, kpos = k, v, np.asarray(pos)
    o = causal_softmax_attention(q, k_all, v_all, np.asarray(pos), kpos, float(m["scale"]), float(m.get("softcap") or 0.0))
    o = o.reshape(T, H * Dv) * sigmoid(h @ p["g"].T)
    return o @ p["o"].T + p["o.b"], dict(k=k_all, v=v_all, kpos=kpos, tails=tails)


def exp_gates(h, p, cap):
    """-> log input gate i [T, H] and log forget gate f [T, H]."""
    zi = h @ p["i"].T + p["i.b"]
    zf = h @ p["f"].T + p["f.b"]
    return cap * np.tanh(zi / cap), logsigmoid(cap * np.tanh(zf / cap))


def matrix_memory_step(S, n, m, q, k, v, i, f):
    """One token of one head: S [D, Dv], n [D], m scalar. -> o [Dv], S', n', m'"""
    m2 = max(f + m, i)
    a, b = math.exp(f + m - m2), math.exp(i - m2)
    S2 = a * S + b * np.outer(k, v)
    n2 = a * n + b * k
    den = max(abs(float(n2 @ q)), math.exp(-m2)) + 1e-6
    return (S2.T @ q) / den, S2, n2, m2


def memory_branch(h, p, m, eps, state=None):
    """The right mixer.  state = dict(S [H, D, Dv], n [H, D], m [H]). -> output [T, W] and the new state."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    if state is None:
        state = dict(S=np.zeros((H, D, Dv), F), n=np.zeros((H, D), F), m=np.zeros(H, F))
    S, n, mm = state["S"].copy(), state["n"].copy(), state["m"].copy()
    q = (h @ p["q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ p["k"].T).reshape(T, H, D)
    v = (h @ p["v"].T).reshape(T, H, Dv)
    gi, gf = exp_gates(h, p, float(m["gate_cap"]))
    o = np.zeros((T, H, Dv), F)
    for t in range(T):
        for hd in range(H):
            o[t, hd], S[hd], n[hd], mm[hd] = matrix_memory_step(S[hd], n[hd], mm[hd], q[t, hd], k[t, hd], v[t, hd], gi[t, hd], gf[t, hd])
    o = rms_unit(o, eps).reshape(T, H * Dv) * p["norm"] * sigmoid(h @ p["g"].T)
    return o @ p["o"].T, dict(S=S, n=n, m=mm)


def split_prefixed(p, prefix):
    return {k[len(prefix):]: v for k, v in p.items() if k.startswith(prefix)}


def parallel_mixer(h, p, m, eps, pos, state=None):
    state = state or {}
    yl, sl = attention_branch(h, split_prefixed(p, "left."), m["left"], pos, state.get("left"))
    yr, sr = memory_branch(h, split_prefixed(p, "right."), m["right"], eps, state.get("right"))
    return float(m["left_scale"]) * yl + float(m["right_scale"]) * yr, dict(left=sl, right=sr)


def ssm_step(S, x, B, C, dt, A_log, Dskip):
    """One token of one head: S [N, Dv]. -> y [Dv], S'"""
    S2 = math.exp(-math.exp(A_log) * dt) * S + dt * np.outer(B, x)
    return S2.T @ C + Dskip * x, S2


def grouped_rms(y, parts, eps):
    """y [T, n] divided, in `parts` equal pieces, by each piece's root mean square."""
    T, n = y.shape
    return rms_unit(y.reshape(T, parts, n // parts), eps).reshape(T, n)


def mamba2_mixer(h, p, m, eps, state=None):
    """state = dict(S [H, N, Dv], tail). -> output [T, W] and the new state."""
    T = h.shape[0]
    H, Dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * Dv
    state = state or {}
    S = state["S"].copy() if "S" in state else np.zeros((H, N, Dv), F)
    zx = h @ p["in"].T
    z, xbc, dt = zx[:, :inner], zx[:, inner:2 * inner + 2 * G * N], zx[:, 2 * inner + 2 * G * N:]
    xbc, tail = short_conv(xbc, p["conv"], state.get("tail"))
    xbc = silu(xbc + p["conv.b"])
    x = xbc[:, :inner].reshape(T, H, Dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + p["dt_bias"])
    y = np.zeros((T, H, Dv), F)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            y[t, hd], S[hd] = ssm_step(S[hd], x[t, hd], B[t, g], C[t, g], dt[t, hd], float(p["A_log"][hd]), float(p["D"][hd]))
    y = grouped_rms(y.reshape(T, inner) * silu(z), int(m["norm_groups"]), eps) * p["norm"]
    return y @ p["o"].T, dict(S=S, tail=tail)


def relu2_ff(h, p):
    return np.maximum(h @ p["up"].T, 0.0) ** 2 @ p["down"].T


def split_params(sd, n_layers):
    """Flat {name: array} -> per-layer dictionaries of float64 arrays (mix / mlp / norms)."""
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
                mlp[rest[4:]] = g(k)
            else:
                norms[rest] = g(k)
        layers.append(dict(mix=mix, mlp=mlp, norms=norms))
    return dict(embed=g("embed"), embed_norm=g("embed.norm"), final_norm=g("final.norm"), layers=layers)


class FunudraOracle:
    """The decoder over a checkpoint, fed in portions.  A sequence's state: per layer (shared weights or not) its own keys,
    values, convolution tails and recurrent matrices."""

    def __init__(self, cfg, sd):
        self.cfg = cfg
        self.P = split_params(sd, len(cfg["layers"]))
        self.eps = float(cfg["norm"]["eps"])

    def new_state(self):
        return dict(pos=0, layer={})

    def forward(self, tokens, state=None, taps=None):
        """The next tokens of one sequence -> logits [T, vocab].  taps (a list) receives the stream after every layer."""
        cfg, P, eps = self.cfg, self.P, self.eps
        st = state if state is not None else self.new_state()
        T = len(tokens)
        pos = st["pos"] + np.arange(T)
        x = rms_norm(P["embed"][np.asarray(tokens)], P["embed_norm"], eps)
        for i, ly in enumerate(cfg["layers"]):
            src = i
            while cfg["layers"][src].get("weights_of") is not None:  # the tensors' owner may itself stand anywhere in the list
                src = int(cfg["layers"][src]["weights_of"])
            p = P["layers"][src]
            h = rms_norm(x, p["norms"]["norm1"], eps)
            if ly["type"] == "mamba2":
                y, st["layer"][i] = mamba2_mixer(h, p["mix"], ly["mixer"], eps, st["layer"].get(i))
            elif ly["type"] == "parallel":
                y, st["layer"][i] = parallel_mixer(h, p["mix"], ly["mixer"], eps, pos, st["layer"].get(i))
            elif ly["type"] == "attention":  # one of the two mixers alone (tensors mix.*): not a layer of the design, a test's tool
                y, st["layer"][i] = attention_branch(h, p["mix"], ly["mixer"], pos, st["layer"].get(i))
            elif ly["type"] == "memory":
                y, st["layer"][i] = memory_branch(h, p["mix"], ly["mixer"], eps, st["layer"].get(i))
            else:
                raise ValueError(ly["type"])
            if ly.get("mlp"):
                y = y + relu2_ff(rms_norm(x, p["norms"]["norm2"], eps), p["mlp"])
            x = x + y
            if taps is not None:
                taps.append(x.copy())
        st["pos"] += T
        return rms_norm(x, P["final_norm"], eps) @ P["embed"].T

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
    return FunudraOracle(cfg, sd).forward(tokens, taps=trace)


# ------------------------------------------------------------------ random checkpoints for tests
def mamba2_cfg(heads=4, vdim=8, state=8, groups=2, norm_groups=2, conv=4):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=norm_groups, conv=conv)


def parallel_cfg(heads=4, kv_heads=2, dim=8, vdim=12, conv=3, rot_dims=4, base=100.0, factor=1.5, scale=None, softcap=8.0,
                 r_heads=3, r_dim=8, r_vdim=8, gate_cap=6.0, left_scale=0.7, right_scale=0.6):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, scale=float(scale if scale is not None else dim ** -0.5),
                softcap=float(softcap))
    if rot_dims:
        left["rot"] = dict(dims=rot_dims, base=float(base))
        if factor:
            left["rot"]["scaling"] = dict(factor=float(factor))
    return dict(left=left, right=dict(heads=r_heads, dim=r_dim, vdim=r_vdim, gate_cap=float(gate_cap)),
                left_scale=float(left_scale), right_scale=float(right_scale))


def random_config(width=48, vocab=90, order=(("mamba2", True), ("parallel", True), ("mamba2", False)), shared=None, ff=64,
                  eps=1e-5, mamba2=None, parallel=None, per_layer=None):
    """order: (type, has feed-forward) per layer; shared {i: j}: layer i uses layer j's tensors; per_layer {i: mixer dict}."""
    layers = []
    for i, (kind, has_ff) in enumerate(order):
        mixer = dict(mamba2 or mamba2_cfg()) if kind == "mamba2" else copy.deepcopy(parallel or parallel_cfg())
        if kind == "attention":
            mixer = mixer["left"]
        elif kind == "memory":
            mixer = mixer["right"]
        if per_layer and i in per_layer:
            mixer = per_layer[i]
        ly = dict(type=kind, mixer=mixer, mlp=dict(kind="dense", ff=ff) if has_ff else None)
        layers.append(ly)
    for i, j in (shared or {}).items():
        layers[i] = dict(layers[j], weights_of=j)
    return dict(architecture="Funudra", width=width, vocab=vocab, layers=layers, norm=dict(eps=eps))


def random_state_dict(cfg, seed=0):
    from .weights import _t
    W, V = cfg["width"], cfg["vocab"]
    s = lambda n: 1.0 / math.sqrt(n)
    sd = {"embed": _t(seed, "embed", (V, W), 0.5), "embed.norm": _t(seed, "en", (W,), 0.1, 1.0),
          "final.norm": _t(seed, "fn", (W,), 0.1, 1.0)}
    for i, ly in enumerate(cfg["layers"]):
        if ly.get("weights_of") is not None:
            continue
        m, p = ly["mixer"], f"l{i}."
        sd[p + "norm1"] = _t(seed, p + "n1", (W,), 0.1, 1.0)
        if ly["type"] == "mamba2":
            H, Dv, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, C = H * Dv, H * Dv + 2 * G * N
            sd[p + "mix.in"] = _t(seed, p + "in", (2 * inner + 2 * G * N + H, W), 1.5 * s(W))
            sd[p + "mix.conv"] = _t(seed, p + "c", (C, taps), 0.5)
            sd[p + "mix.conv.b"] = _t(seed, p + "cb", (C,), 0.2)
            sd[p + "mix.dt_bias"] = _t(seed, p + "dt", (H,), 0.5, -1.0)
            sd[p + "mix.A_log"] = _t(seed, p + "A", (H,), 0.5, -1.0)
            sd[p + "mix.D"] = _t(seed, p + "D", (H,), 0.3, 1.0)
            sd[p + "mix.norm"] = _t(seed, p + "hn", (inner,), 0.1, 1.0)
            sd[p + "mix.o"] = _t(seed, p + "o", (W, inner), s(inner))
        else:
            if ly["type"] in ("parallel", "attention"):
                l, q = (m["left"], p + "mix.left.") if ly["type"] == "parallel" else (m, p + "mix.")
                H, G, D, Dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
                for n, rows in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                    sd[q + n] = _t(seed, q + n, (rows, W), 1.5 * s(W))
                    sd[q + n + ".b"] = _t(seed, q + n + "b", (rows,), 0.2)
                    if l.get("conv"):
                        sd[q + n + ".conv"] = _t(seed, q + n + "c", (rows, l["conv"]), 0.5)
                sd[q + "g"] = _t(seed, q + "g", (H * Dv, W), 1.5 * s(W))
                sd[q + "o"] = _t(seed, q + "o", (W, H * Dv), s(H * Dv))
                sd[q + "o.b"] = _t(seed, q + "ob", (W,), 0.1)
            if ly["type"] in ("parallel", "memory"):
                r, q = (m["right"], p + "mix.right.") if ly["type"] == "parallel" else (m, p + "mix.")
                H, D, Dv = r["heads"], r["dim"], r["vdim"]
                sd[q + "q"] = _t(seed, q + "q", (H * D, W), 1.5 * s(W))
                sd[q + "k"] = _t(seed, q + "k", (H * D, W), 1.5 * s(W))
                sd[q + "v"] = _t(seed, q + "v", (H * Dv, W), 1.5 * s(W))
                sd[q + "g"] = _t(seed, q + "g", (H * Dv, W), 1.5 * s(W))
                sd[q + "o"] = _t(seed, q + "o", (W, H * Dv), s(H * Dv))
                sd[q + "norm"] = _t(seed, q + "n", (H * Dv,), 0.1, 1.0)
                sd[q + "i"] = _t(seed, q + "i", (H, W), 2.0 * s(W))
                sd[q + "i.b"] = _t(seed, q + "ib", (H,), 0.5)
                sd[q + "f"] = _t(seed, q + "f", (H, W), 2.0 * s(W))
                sd[q + "f.b"] = _t(seed, q + "fb", (H,), 0.5, 2.0)
        if ly.get("mlp"):
            Fn = ly["mlp"]["ff"]
            sd[p + "norm2"] = _t(seed, p + "n2", (W,), 0.1, 1.0)
            sd[p + "mlp.up"] = _t(seed, p + "u", (Fn, W), 1.5 * s(W))
            sd[p + "mlp.down"] = _t(seed, p + "d", (W, Fn), s(Fn))
    return sd
