"""CPU checks of the Latanex oracle (float64) against closed forms, and of the configuration reader: no GPU, no library calls."""
import math

import numpy as np
import pytest

from helix_b200 import weights_io
from helix_b200 import engine as E
from oracle import latanex_ref as ref


def test_oracle_portions_equal_whole():
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=2)
    o = ref.LatanexOracle(cfg, sd)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 70).tolist()
    whole = o.forward(toks)
    assert np.abs(whole - ref.forward(cfg, sd, toks)).max() == 0.0
    st, parts, at = o.new_state(), [], 0
    for n in (19, 2, 1, 30, 18):
        parts.append(o.forward(toks[at:at + n], st))
        at += n
    assert np.abs(np.concatenate(parts) - whole).max() < 1e-9


def test_tanh_norm_is_element_wise():
    p = {"n": np.array([2.0, -1.0]), "n.b": np.array([0.5, 0.25]), "n.alpha": np.array(0.5)}
    x = np.array([[1.0, 4.0], [100.0, -100.0]])
    y = ref.tanh_norm(x, p, "n")
    assert np.allclose(y[0], [2.0 * math.tanh(0.5) + 0.5, -math.tanh(2.0) + 0.25])
    assert np.allclose(y[1], [2.5, 1.25])  # saturates: no statistic of the row enters


def test_window_sink_and_cap_by_construction():
    # zero queries (zero weights, zero bias): every visible key scores 0, so with a sink of 0 the weights are 1 / (visible + 1);
    # values planted so that token j carries j + 1
    H, G, D, Dv, Wd, T, size = 2, 1, 2, 1, 3, 9, 4
    m = dict(heads=H, kv_heads=G, dim=D, vdim=Dv, scale=1.0, mask=dict(size=size), softcap=5.0, v_mix=False)
    p = {"q": np.zeros((H * D, Wd)), "q.b": np.zeros(H * D), "k": np.ones((G * D, Wd)), "k.b": np.zeros(G * D), "v": np.array([[1.0, 0, 0]]),
         "v.b": np.zeros(1), "q.norm": np.ones(H * D), "k.norm": np.ones(G * D), "sink": np.array([0.0, math.log(3.0)]), "o": np.eye(Wd, H * Dv)}
    h = np.zeros((T, Wd))
    h[:, 0] = np.arange(1, T + 1)
    out, (k, v, kpos), _ = ref.attention_mixer(h, p, m, 1e-6)
    for t in range(T):
        vis = [j for j in range(T) if 0 <= t - j < size]
        assert vis == [j for j in range(T) if ref.window_visible(t, j, size)]
        assert out[t, 0] == pytest.approx(sum(j + 1 for j in vis) / (len(vis) + 1))   # sink 0 counts as one key of score 0
        assert out[t, 1] == pytest.approx(sum(j + 1 for j in vis) / (len(vis) + 3))   # exp(sink) = 3, unscaled, once
    assert len([j for j in range(T) if ref.window_visible(T - 1, j, size)]) == size
    out2, _, _ = ref.attention_mixer(h, p, dict(m, mask=None), 1e-6)                # no mask key: causal
    assert out2[T - 1, 0] == pytest.approx(sum(range(1, T + 1)) / (T + 1))
    assert ref.capped(np.array([1e9, -1e9, 0.1]), 5.0) == pytest.approx([5.0, -5.0, 5.0 * math.tanh(0.02)])
    assert ref.capped(np.array([7.0]), 0)[0] == 7.0


def test_q_and_k_are_normed_over_the_whole_projection():
    rng = np.random.default_rng(3)
    m = dict(heads=3, kv_heads=1, dim=4, vdim=2)
    p = {n: rng.standard_normal(s) for n, s in (("q", (12, 5)), ("q.b", 12), ("k", (4, 5)), ("k.b", 4), ("v", (2, 5)), ("v.b", 2))}
    p["q.norm"], p["k.norm"] = np.ones(12), np.full(4, 2.0)
    h = rng.standard_normal((6, 5))
    q, k, v = ref.attention_qkv(h, p, m, 0.0)
    assert np.allclose((q.reshape(6, -1) ** 2).mean(-1), 1.0)        # one statistic for all heads ...
    assert not np.allclose((q ** 2).mean(-1), 1.0)                   # ... not one per head
    assert np.allclose((k.reshape(6, -1) ** 2).mean(-1), 4.0)
    assert np.allclose(v.reshape(6, -1), h @ p["v"].T + p["v.b"])


def test_blended_values():
    v, vf = np.array([1.0, 2.0]), np.array([3.0, -2.0])
    assert np.allclose(ref.blend_values(v, vf, 0.25), [1.5, 1.0])
    assert ref.blend_values(v, None, 0.25) is v


def test_short_convolution_and_its_tail():
    rng = np.random.default_rng(4)
    x, w = rng.standard_normal((10, 3)), rng.standard_normal((3, 4))
    y, tail = ref.short_conv(x, w)
    assert y[0] == pytest.approx(x[0] * w[:, 3])                                    # zeros before the start
    assert y[5] == pytest.approx(x[2] * w[:, 0] + x[3] * w[:, 1] + x[4] * w[:, 2] + x[5] * w[:, 3])
    assert np.array_equal(tail, x[7:])
    parts, t = [], None
    for a, b in ((0, 1), (1, 3), (3, 4), (4, 10)):  # portions shorter than the taps
        yy, t = ref.short_conv(x[a:b], w, t)
        parts.append(yy)
    assert np.allclose(np.concatenate(parts), y) and np.allclose(t, tail)
    y1, t1 = ref.short_conv(x, w[:, 3:])  # one tap: no tail
    assert np.allclose(y1, x * w[:, 3]) and t1.shape == (0, 3)


def test_delta_rule_stores_and_overwrites():
    # orthonormal keys, beta = 1, no decay: the state returns each stored value exactly; writing a key again replaces its value
    D, Dv = 4, 3
    rng = np.random.default_rng(5)
    keys, vals = np.eye(D), rng.standard_normal((D, Dv))
    S = np.zeros((D, Dv))
    for i in range(D):
        S, o = ref.delta_step(S, keys[i], keys[i], vals[i], 1.0, 1.0)
        assert np.allclose(o, vals[i])                       # the read-out sees the current write
    assert np.allclose(S, vals)
    S, o = ref.delta_step(S, keys[0], keys[1], np.ones(Dv), 1.0, 1.0)
    assert np.allclose(S[1], 1.0) and np.allclose(o, vals[0])
    S2, _ = ref.delta_step(vals.copy(), keys[0], keys[1], np.ones(Dv), 0.5, 0.5)  # decay first, then half of the error
    assert np.allclose(S2[1], 0.5 * vals[1] + 0.5 * (1.0 - 0.5 * vals[1])) and np.allclose(S2[0], 0.5 * vals[0])
    assert np.allclose(ref.unit_vector(np.array([3.0, 4.0])), [0.6, 0.8], atol=1e-6)
    assert ref.softplus(np.array([-800.0, 0.0, 800.0])) == pytest.approx([0.0, math.log(2.0), 800.0])


def test_router_groups_by_construction():
    # 6 experts in 3 groups of 2; a zero router gives every score 1/2, the corrections decide
    r = dict(experts=6, top=2, scale=3.0, groups=dict(count=3, keep=1))
    p = {"router": np.zeros((6, 4)), "correction": np.array([0.3, 0.0, 0.2, 0.2, 0.35, -0.9])}
    h = np.ones((1, 4))
    idx, wt = ref.moe_route(h, p, r)
    # group sums of the two largest: 1.3, 1.4, 0.45 -> only group 1 stays, although expert 4 has the largest single score
    assert sorted(idx[0]) == [2, 3] and np.allclose(wt, 1.5)
    idx, _ = ref.moe_route(h, p, dict(r, groups=dict(count=3, keep=2)))
    assert sorted(idx[0]) == [0, 2]                                  # ties go to the lower index
    idx, wt = ref.moe_route(h, p, dict(experts=6, top=3, scale=1.0))
    assert list(idx[0]) == [4, 0, 2] and np.allclose(wt, 1.0 / 3)
    p["correction"] = np.array([-5.0, -5.0, -3.0, -9.0, -4.0, -4.5])  # negative choice scores: dropped groups are -inf, not 0
    idx, _ = ref.moe_route(h, p, r)
    assert sorted(idx[0]) == [4, 5]
    assert ref.route_margin(h, p, r)[0] == pytest.approx(1.5)  # group sums -9, -11, -7.5: the edge between groups 2 and 0 decides


def test_clamped_expert():
    p = {"gate": np.array([[1.0], [1.0]]), "up": np.array([[1.0], [-1.0]]), "down": np.eye(2)}
    y = ref.clamped_expert(np.array([[10.0]]), p, 2.0)   # gate clamps from above only, up on both sides
    g = 2.0 / (1.0 + math.exp(-1.702 * 2.0))
    assert np.allclose(y, [[g * 3.0, g * -1.0]])
    y = ref.clamped_expert(np.array([[-10.0]]), p, 2.0)
    g = -10.0 / (1.0 + math.exp(17.02))
    assert np.allclose(y, [[g * -1.0, g * 3.0]])


def test_config_reader_maps_every_key():
    cfg = ref.random_config(order=(("attention", "dense"), ("delta", "moe"), ("attention", None)),
                            per_layer={2: dict(v_mix=False, softcap=None, mask=None)})
    d = weights_io.desc_from_hf_config(cfg, compute_f32=True)
    assert isinstance(d, E.StackDesc) and d.compute_f32 == 1
    assert (d.width, d.vocab, len(d.layers)) == (cfg["width"], cfg["vocab"], 3)
    assert d.norm_place == E.NORM_BOTH_SIDES and d.norm_kind == E.NORM_TANH and d.plain_gains == 1 and d.embed_norm == 0
    assert d.embed_scale == 2.0 and d.logit_scale == 0.5 and d.norm_eps == pytest.approx(1e-5)
    a, dl, c = d.layers
    m = cfg["layers"][0]["mixer"]
    assert a.mixer == E.MIXER_GQA and (a.heads, a.kv_heads, a.dim, a.vdim) == (m["heads"], m["kv_heads"], m["dim"], m["vdim"])
    assert a.attn_flags == E.ATTN_QKV_BIAS | E.ATTN_QK_PROJ_NORM | E.ATTN_LEARNED_SINK | E.ATTN_V_BLEND
    assert a.mask == E.MASK_WINDOW and a.window == m["mask"]["size"] and a.score_cap == m["softcap"] and a.scale == pytest.approx(m["scale"])
    assert a.rope_dims == 0 and a.ff_kind == E.FF_SILU and a.ff == cfg["layers"][0]["mlp"]["ff"]
    assert c.attn_flags == E.ATTN_QKV_BIAS | E.ATTN_QK_PROJ_NORM | E.ATTN_LEARNED_SINK and c.mask == E.MASK_CAUSAL and c.score_cap == 0.0 and c.ff == 0
    m, mlp = cfg["layers"][1]["mixer"], cfg["layers"][1]["mlp"]
    assert dl.mixer == E.MIXER_DELTA and (dl.heads, dl.kv_heads, dl.dim, dl.vdim, dl.conv_taps) == (m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"])
    assert dl.ff_kind == E.FF_MOE and dl.ff == mlp["expert"]["ff"] and dl.ff_limit == mlp["expert"]["limit"]
    assert (dl.experts, dl.top_k, dl.identity_experts) == (mlp["router"]["experts"], mlp["router"]["top"], 0)
    assert dl.router_kind == E.ROUTER_SIGMOID and dl.expert_kind == E.EXPERT_CLAMPED and dl.route_renorm == 1
    assert (dl.route_groups, dl.route_keep, dl.route_scale) == (3, 2, 1.5)
    assert (dl.shared_ff, dl.shared_limit) == (mlp["shared"]["ff"], mlp["shared"]["limit"])
    bare = ref.random_config(order=(("delta", "moe"),), groups=None, shared_ff=0)
    del bare["embedding"], bare["logit_scale"], bare["layers"][0]["mlp"]["router"]["scale"]
    b = weights_io.desc_from_hf_config(bare)
    assert b.embed_scale == 1.0 and b.logit_scale == 1.0 and b.layers[0].route_groups == 0 and b.layers[0].shared_ff == 0
    assert b.layers[0].route_scale == 1.0 and b.compute_f32 == 0
    with pytest.raises(ValueError):
        weights_io.desc_from_hf_config(dict(cfg, layers=[dict(cfg["layers"][0], type="conv")]))
    # the C mirror carries every field
    sd, arr = d.to_c()
    assert (sd.norm_kind, sd.norm_place, sd.embed_scale, sd.logit_scale) == (E.NORM_TANH, E.NORM_BOTH_SIDES, 2.0, 0.5)
    assert (arr[1].conv_taps, arr[1].route_groups, arr[1].route_keep, arr[1].shared_ff, arr[1].expert_kind) == (4, 3, 2, 48, E.EXPERT_CLAMPED)
    assert arr[0].score_cap == 6.0 and arr[0].attn_flags == a.attn_flags
