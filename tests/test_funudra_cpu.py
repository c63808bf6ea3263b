"""CPU: the float64 Funudra oracle against closed forms written out by hand, its own state handling under portions, and the
configuration reader key by key.  The engine is compared with this oracle in tests/test_funudra_gpu.py."""
import copy
import math

import numpy as np
import pytest

from helix_b200 import engine as E
from helix_b200 import weights_io
from oracle import funudra_ref as ref


def rnd(seed, *shape):
    return np.random.default_rng(seed).standard_normal(shape)


def test_short_convolution_taps_order_zero_start_and_tails():
    u, w = rnd(0, 9, 3), rnd(1, 3, 4)
    y, tail = ref.short_conv(u, w)
    # the last column multiplies the current token, the first one the token three back; nothing before the start
    assert np.allclose(y[0], w[:, 3] * u[0])
    assert np.allclose(y[5], w[:, 0] * u[2] + w[:, 1] * u[3] + w[:, 2] * u[4] + w[:, 3] * u[5])
    assert np.array_equal(tail, u[-3:])
    # portions shorter than the taps: the tail is made of old and new inputs
    t, out = None, []
    for a, b in ((0, 2), (2, 3), (3, 4), (4, 9)):
        o, t = ref.short_conv(u[a:b], w, t)
        out.append(o)
    assert np.allclose(np.concatenate(out), y)
    one, t1 = ref.short_conv(u, rnd(2, 3, 1))  # a single tap keeps no tail
    assert t1.shape == (0, 3)


def test_rotation_pairs_halves_scales_linearly_and_keeps_the_rest():
    x = rnd(3, 5, 2, 10)
    pos = np.array([0, 1, 7, 100, 1000])
    y = ref.rotate_half_layout(x, pos, 6, 50.0, 2.0)
    assert np.array_equal(y[..., 6:], x[..., 6:]) and np.allclose(y[0], x[0])
    for i in range(3):  # entry i turns with entry i + 3 by pos * base^(-2i/6) / 2
        a = pos * 50.0 ** (-2.0 * i / 6) / 2.0
        assert np.allclose(y[:, 1, i], x[:, 1, i] * np.cos(a) - x[:, 1, i + 3] * np.sin(a))
        assert np.allclose(y[:, 1, i + 3], x[:, 1, i + 3] * np.cos(a) + x[:, 1, i] * np.sin(a))
    # neighbouring pairs (2i, 2i + 1) would be another model; so would an unscaled frequency
    assert np.abs(ref.rotate_half_layout(x, pos, 6, 50.0, 1.0) - y).max() > 0.1
    # scores depend on the distance only
    q, k = rnd(4, 1, 1, 6), rnd(5, 1, 1, 6)
    s = lambda pq, pk: float(ref.rotate_half_layout(q, [pq], 6, 50.0, 2.0)[0, 0] @ ref.rotate_half_layout(k, [pk], 6, 50.0, 2.0)[0, 0])
    assert abs(s(40, 33) - s(1007, 1000)) < 1e-9


def test_attention_cap_causality_and_groups():
    q, k, v = rnd(6, 4, 4, 3), rnd(7, 4, 2, 3), rnd(8, 4, 2, 5)
    pos = np.arange(4)
    o = ref.causal_softmax_attention(q, k, v, pos, pos, 0.7, 2.0)
    assert np.allclose(o[0, 3], v[0, 1])  # the first position sees itself only; head 3 reads key/value head 1
    s = 2.0 * np.tanh(0.7 * (q[2, 1] @ k[:3, 0].T) / 2.0)
    p = np.exp(s) / np.exp(s).sum()
    assert np.allclose(o[2, 1], p @ v[:3, 0])
    assert np.abs(ref.causal_softmax_attention(q, k, v, pos, pos, 0.7, 0.0) - o).max() > 1e-3


def test_matrix_memory_running_maximum_starts_at_zero():
    D, Dv = 3, 2
    S, n = np.zeros((D, Dv)), np.zeros(D)
    q, k, v = np.array([1.0, 0.0, 0.0]), np.array([2.0, 0.0, 0.0]), np.array([3.0, -1.0])
    # i = -3, f = -0.1: m' = max(-0.1 + 0, -3) = -0.1 (from minus infinity it would be -3)
    o, S1, n1, m1 = ref.matrix_memory_step(S, n, 0.0, q, k, v, -3.0, -0.1)
    assert m1 == -0.1
    b = math.exp(-3.0 + 0.1)
    assert np.allclose(S1[0], b * 2.0 * v) and np.allclose(n1, b * k)
    assert np.allclose(o, b * 2.0 * v / (max(abs(b * 2.0), math.exp(0.1)) + 1e-6))
    # the stabilised recurrence equals the plain sums: S = sum_s exp(i_s + sum_{r > s} f_r) k_s v_s^T
    T = 12
    qs, ks, vs = rnd(9, T, D), rnd(10, T, D), rnd(11, T, Dv)
    gi, gf = rnd(12, T) * 2.0, -np.abs(rnd(13, T))
    S, n, m = np.zeros((D, Dv)), np.zeros(D), 0.0
    for t in range(T):
        o, S, n, m = ref.matrix_memory_step(S, n, m, qs[t], ks[t], vs[t], gi[t], gf[t])
        w = np.array([math.exp(gi[s] + gf[s + 1:t + 1].sum()) for s in range(t + 1)])
        S_plain = np.einsum("s,sd,se->de", w, ks[:t + 1], vs[:t + 1])
        n_plain = w @ ks[:t + 1]
        assert np.allclose(S * math.exp(m), S_plain) and np.allclose(n * math.exp(m), n_plain)
        assert abs(m - max(gf[:t + 1].sum(), max(gi[s] + gf[s + 1:t + 1].sum() for s in range(t + 1)))) < 1e-12
        assert np.allclose(o, S_plain.T @ qs[t] * math.exp(-m) / (max(abs(n_plain @ qs[t]) * math.exp(-m), math.exp(-m)) + 1e-6))


def test_gates_cap_and_log_sigmoid():
    p = {"i": np.zeros((2, 3)), "f": np.zeros((2, 3)), "i.b": np.array([100.0, -0.5]), "f.b": np.array([-100.0, 0.5])}
    gi, gf = ref.exp_gates(np.zeros((1, 3)), p, 4.0)
    assert np.allclose(gi[0], [4.0, 4.0 * math.tanh(-0.125)])
    assert np.allclose(gf[0], [math.log(1.0 / (1.0 + math.exp(4.0))), math.log(1.0 / (1.0 + math.exp(-4.0 * math.tanh(0.125))))])


def test_state_space_step_and_grouped_norm():
    N, Dv, T = 3, 2, 7
    xs, Bs, Cs, dt = rnd(14, T, Dv), rnd(15, T, N), rnd(16, T, N), np.abs(rnd(17, T)) + 0.1
    A_log, D = -0.3, 0.7
    S = np.zeros((N, Dv))
    for t in range(T):
        y, S = ref.ssm_step(S, xs[t], Bs[t], Cs[t], dt[t], A_log, D)
        a = np.exp(-math.exp(A_log) * dt)
        S_plain = sum(np.prod(a[s + 1:t + 1]) * dt[s] * np.outer(Bs[s], xs[s]) for s in range(t + 1))
        assert np.allclose(S, S_plain) and np.allclose(y, S_plain.T @ Cs[t] + D * xs[t])
    y = rnd(18, 2, 12)
    g = ref.grouped_rms(y, 3, 1e-6)
    assert np.allclose((g.reshape(2, 3, 4) ** 2).mean(-1), 1.0, atol=1e-4)
    assert np.abs(ref.grouped_rms(y, 1, 1e-6) - g).max() > 1e-2
    assert np.allclose(ref.relu2_ff(np.array([[1.0, -2.0]]), {"up": np.array([[1.0, 0.0], [0.0, 1.0]]), "down": np.array([[1.0, 5.0]])}), [[1.0]])


def test_mamba2_layout_gate_before_norm_and_softplus_without_clamp():
    cfg = ref.random_config(order=(("mamba2", False),), mamba2=ref.mamba2_cfg(heads=2, vdim=4, state=3, groups=1, norm_groups=2, conv=2))
    sd = ref.random_state_dict(cfg, seed=1)
    m = cfg["layers"][0]["mixer"]
    p = ref.split_params(sd, 1)["layers"][0]["mix"]
    h = rnd(19, 6, cfg["width"])
    y, st = ref.mamba2_mixer(h, p, m, 1e-5)
    # by hand: [z | x | B | C | dt] = 8 | 8 | 3 | 3 | 2 rows
    zx = h @ p["in"].T
    z, xbc, dt = zx[:, :8], zx[:, 8:22], zx[:, 22:]
    conv, _ = ref.short_conv(xbc, p["conv"])
    xbc = ref.silu(conv + p["conv.b"])
    dt = np.log1p(np.exp(dt + p["dt_bias"]))
    S = np.zeros((2, 3, 4))
    rows = []
    for t in range(6):
        o = []
        for hd in range(2):
            x = xbc[t, 4 * hd:4 * hd + 4]
            S[hd] = math.exp(-math.exp(p["A_log"][hd]) * dt[t, hd]) * S[hd] + dt[t, hd] * np.outer(xbc[t, 8:11], x)
            o.append(S[hd].T @ xbc[t, 11:14] + p["D"][hd] * x)
        u = np.concatenate(o) * ref.silu(z[t])
        u = np.concatenate([u[:4] / math.sqrt((u[:4] ** 2).mean() + 1e-5), u[4:] / math.sqrt((u[4:] ** 2).mean() + 1e-5)])
        rows.append((u * p["norm"]) @ p["o"].T)
    assert np.allclose(np.stack(rows), y)
    assert np.allclose(st["S"], S) and np.array_equal(st["tail"], (zx[:, 8:22])[-1:])


def test_portions_and_shared_tensors_in_the_oracle():
    cfg = ref.random_config(order=(("mamba2", True), ("parallel", True), ("mamba2", False), ("parallel", False)), shared={2: 0, 3: 1})
    cfg["layers"][2]["mlp"] = cfg["layers"][0]["mlp"]
    sd = ref.random_state_dict(cfg, seed=2)
    assert not any(k.startswith(("l2.", "l3.")) for k in sd)
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], 40).tolist()
    o = ref.FunudraOracle(cfg, sd)
    want = o.forward(toks)
    st, out = o.new_state(), []
    for a, b in ((0, 1), (1, 3), (3, 4), (4, 21), (21, 23), (23, 40)):
        out.append(o.forward(toks[a:b], st))
    assert np.allclose(np.concatenate(out), want, atol=1e-9)
    # the same model with copies of the tensors instead of references
    own = copy.deepcopy(cfg)
    sd2 = dict(sd)
    for i, j in ((2, 0), (3, 1)):
        del own["layers"][i]["weights_of"]
        for k, v in sd.items():
            if k.startswith(f"l{j}."):
                sd2[f"l{i}." + k[len(f"l{j}."):]] = v
    assert np.allclose(ref.FunudraOracle(own, sd2).forward(toks), want, atol=1e-12)
    # the owner of the tensors may stand behind its user, and a user may name another user
    later = copy.deepcopy(own)
    later["layers"][0]["weights_of"] = 2
    later["layers"][3]["weights_of"] = 1
    sd3 = {k: v for k, v in sd2.items() if not k.startswith(("l0.", "l3."))}
    assert np.allclose(ref.FunudraOracle(later, sd3).forward(toks), want, atol=1e-12)
    d = weights_io.desc_from_hf_config(later)
    assert [l.weights_of for l in d.layers] == [3, 0, 0, 2]
    chain = copy.deepcopy(cfg)
    chain["layers"][3]["weights_of"] = 1
    chain["layers"].append(dict(chain["layers"][3], weights_of=3))
    assert [l.weights_of for l in weights_io.desc_from_hf_config(chain).layers] == [0, 0, 1, 2, 2]
    # the output matrix is the embedding table, after the final norm
    taps = []
    o.forward(toks, taps=taps)
    assert np.allclose(ref.rms_norm(taps[-1], sd["final.norm"], 1e-5) @ np.asarray(sd["embed"], float).T, want)


def test_both_sublayers_read_the_same_stream():
    cfg = ref.random_config(order=(("parallel", True),))
    sd = ref.random_state_dict(cfg, seed=3)
    o = ref.FunudraOracle(cfg, sd)
    toks = [3, 9, 27, 5]
    taps = []
    o.forward(toks, taps=taps)
    P = o.P["layers"][0]
    x0 = ref.rms_norm(np.asarray(sd["embed"], float)[toks], sd["embed.norm"], 1e-5)
    mix, _ = ref.parallel_mixer(ref.rms_norm(x0, P["norms"]["norm1"], 1e-5), P["mix"], cfg["layers"][0]["mixer"], 1e-5, np.arange(4))
    ff = ref.relu2_ff(ref.rms_norm(x0, P["norms"]["norm2"], 1e-5), P["mlp"])
    assert np.allclose(taps[0], x0 + mix + ff)
    seq = ref.relu2_ff(ref.rms_norm(x0 + mix, P["norms"]["norm2"], 1e-5), P["mlp"])  # a feed-forward behind the mixer is another model
    assert np.abs(seq - ff).max() > 1e-2


def test_configuration_reader_key_by_key():
    par = ref.parallel_cfg(heads=6, kv_heads=3, dim=10, vdim=14, conv=5, rot_dims=8, base=333.0, factor=3.5, scale=0.31, softcap=7.0,
                           r_heads=5, r_dim=12, r_vdim=20, gate_cap=9.0, left_scale=0.4, right_scale=1.3)
    cfg = ref.random_config(width=72, vocab=99, ff=100, eps=3e-5, order=(("mamba2", True), ("parallel", False), ("mamba2", True)), shared={2: 0},
                            mamba2=ref.mamba2_cfg(heads=6, vdim=5, state=7, groups=3, norm_groups=2, conv=3), parallel=par)
    d = weights_io.desc_from_hf_config(cfg, compute_f32=True)
    assert (d.width, d.vocab, d.compute_f32, d.norm_place, d.embed_norm, d.plain_gains, d.tie_head) == (72, 99, 1, E.NORM_PARALLEL, 1, 1, 1)
    assert abs(d.norm_eps - 3e-5) < 1e-12 and d.norm_kind == E.NORM_RMS
    a, b, c = d.layers
    assert (a.mixer, a.heads, a.vdim, a.dim, a.kv_heads, a.norm_groups, a.conv_taps) == (E.MIXER_MAMBA2, 6, 5, 7, 3, 2, 3)
    assert (a.ff_kind, a.ff, a.weights_of) == (E.FF_RELU2, 100, 0)
    assert (b.mixer, b.heads, b.kv_heads, b.dim, b.vdim, b.conv_taps, b.ff) == (E.MIXER_GQA, 6, 3, 10, 14, 5, 0)
    assert b.attn_flags == E.ATTN_QKV_BIAS | E.ATTN_OUT_GATE | E.ATTN_OUT_BIAS | E.ATTN_QKV_CONV
    assert (b.rope_dims, b.rope_pairing, b.mask) == (8, 0, E.MASK_CAUSAL)
    assert (b.rope_base, b.rope_linear, b.scale, b.score_cap) == (333.0, 3.5, 0.31, 7.0)
    assert (b.side_mixer, b.side_heads, b.side_dim, b.side_vdim, b.side_gate_cap) == (E.MIXER_MLSTM, 5, 12, 20, 9.0)
    assert (b.mix_scale, b.side_scale) == (0.4, 1.3)
    assert c.weights_of == 1 and (c.mixer, c.ff) == (a.mixer, a.ff)
    assert d.unused_tensors == frozenset({"l1.norm2"})  # a second norm stored for a layer without a feed-forward is skipped at load
    # absent keys: no convolution, no rotation, no frequency scaling, no cap
    bare = copy.deepcopy(cfg)
    l = bare["layers"][1]["mixer"]["left"]
    del l["conv"], l["softcap"], l["rot"]["scaling"]
    b = weights_io.desc_from_hf_config(bare).layers[1]
    assert not (b.attn_flags & E.ATTN_QKV_CONV) and b.score_cap == 0.0 and b.rope_linear == 0.0 and b.rope_dims == 8
    del l["rot"]
    assert weights_io.desc_from_hf_config(bare).layers[1].rope_dims == 0
    bad = copy.deepcopy(cfg)
    bad["layers"][0]["type"] = "mamba3"
    with pytest.raises(ValueError):
        weights_io.desc_from_hf_config(bad)
