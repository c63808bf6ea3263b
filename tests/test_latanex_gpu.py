"""Latanex layer-list decoders through the engine (driven sequences and the scheduler) against the float64 oracle.

Every test builds its own small configuration and random bf16-representable weights (oracle/latanex_ref.py); the engine runs
them in its exact mode (fp32 weights, cache, state and products), where a window that is one token off, a sink left out, a
lost recurrent state or a wrong expert must show, and in its serving mode (bf16 weights / cache rows / GEMM operands) with a
rounding-sized bound.
"""
import copy

import numpy as np
import pytest

import helix_b200 as hb
from helix_b200 import weights_io
from helix_b200.engine import CAPTURE_PROMPT_LOGITS, CAPTURE_STEP_LOGITS, ATTN_LEARNED_SINK
from oracle import latanex_ref as ref
from oracle.weights import to_bf16_f32

pytestmark = pytest.mark.gpu

TOL = {1: 2e-4, 0: 6e-2}  # compute_f32 -> bound on rms(diff) / rms(expected) per logits row
ATT = (("attention", None),)
DELTA = (("delta", None),)


def row_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    return np.sqrt((d * d).mean(-1)) / np.sqrt((want * want).mean(-1))


def oracle_rows(cfg, sd, toks, f32):
    """Expected logits and the rows a comparison may rest on.  A router's choice between two experts (or groups) whose scores
    nearly tie flips under rounding (serving mode: about 1e-2 of a score).  A flip in the last layer changes that token's row
    only; after a flip in an earlier layer the recurrent layers and the chain of windows carry the difference to every later
    position, so the rows from the first such token on are left out.  The exact mode keeps practically all rows and is the
    sharp test; serving-mode tests that need every row put their mixtures into the last layer or use none."""
    margins = []
    want = ref.LatanexOracle(cfg, sd).forward(toks, margins=margins)
    ok = np.ones(len(toks), bool)
    at = [i for i, ly in enumerate(cfg["layers"]) if ly.get("mlp") and ly["mlp"]["kind"] == "moe"]
    for i, m in zip(at, margins):
        close = np.nonzero(m < (1e-5 if f32 else 3e-2))[0]
        if i == len(cfg["layers"]) - 1:
            ok[close] = False
        elif len(close):
            ok[close[0]:] = False
    return want, ok


def check(got, want, ok, f32, least=0):
    err = row_err(got, want)
    assert ok.sum() >= least, ok.sum()
    assert not ok.any() or err[ok].max() < TOL[f32], (err[ok].max(), int(np.argmax(np.where(ok, err, 0))))
    assert err.max() < 1.5  # a flipped choice changes one unit's output, not the model


def make_engine(cfg, sd, f32, max_seqs=4, ctx=512, pool=0, batched=0, edit=None, **kw):
    desc = weights_io.desc_from_hf_config(copy.deepcopy(cfg), {k: v.shape for k, v in sd.items()}, compute_f32=bool(f32))
    if edit:
        edit(desc)
    e = hb.Engine(hb.EngineConfig(device=0, max_seqs=max_seqs, max_ctx=ctx, max_batched_tokens=batched or ctx,
                                  kv_pool_tokens=pool, **kw))
    e.load_state_dict(desc, sd)
    return e


def tokens(seed, n, vocab):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def replay(e, toks, cuts):
    """Feed one sequence in portions of the given sizes (the rest one token at a time), all positions wanted."""
    sid, out, at = e.seq_open(), [], 0
    cuts = list(cuts)
    while at < len(toks):
        n = min(cuts.pop(0) if cuts else 1, len(toks) - at)
        out.append(e.seq_step([(sid, toks[at:at + n], list(range(n)))]))
        at += n
    e.seq_close(sid)
    return np.concatenate(out)


CONFIGS = {
    "default": dict(),
    "attention_alone": dict(order=ATT),
    "delta_alone": dict(order=DELTA),
    "dense_alone": dict(order=(("attention", "dense"),)),
    "moe_alone": dict(order=(("delta", "moe"),)),
    "moe_last": dict(order=(("attention", "dense"), ("delta", None), ("attention", "moe"))),
    "delta_first_attention_later": dict(order=(("delta", "dense"), ("delta", None), ("attention", "moe"))),
    "one_kv_head": dict(heads=4, kv_heads=1, delta=dict(heads=3, kv_heads=1)),
    "no_grouping": dict(heads=3, kv_heads=3, delta=dict(heads=2, kv_heads=2)),
    "five_heads_per_kv_head": dict(heads=10, kv_heads=2, dim=16, delta=dict(heads=10, kv_heads=2, dim=8, vdim=8)),
    # nothing a multiple of 8 or 4: every product takes the CUDA-core GEMM, rows are loaded element by element
    "odd_sizes": dict(width=90, vocab=131, heads=6, kv_heads=3, dim=14, vdim=10, window=9, ff=50, expert_ff=30, shared_ff=22,
                      delta=dict(heads=6, kv_heads=3, dim=10, vdim=14, conv=3)),
    # values the usual model makes equal or one: equal head sizes, window of one page, no cap, unit scales, one group
    "neutral_constants": dict(dim=16, vdim=16, window=64, softcap=0, embed_scale=1.0, logit_scale=1.0, route_scale=1.0, groups=None,
                              delta=dict(dim=16, vdim=16, conv=1)),
    "causal_no_window": dict(window=0, order=(("attention", "dense"), ("attention", None))),
    "no_blending_and_partial_blending": dict(order=(("attention", None), ("attention", "dense"), ("attention", None), ("attention", None)),
                                             per_layer={0: dict(v_mix=False), 2: dict(v_mix=False)}),
    "layers_differ": dict(order=(("attention", "moe"), ("delta", "dense"), ("attention", None), ("delta", "moe")),
                          per_layer={0: dict(heads=2, kv_heads=1, dim=40, vdim=8, mask=dict(size=7), v_mix=False),
                                     2: dict(heads=8, kv_heads=4, dim=8, vdim=24, softcap=2.0, scale=0.9),
                                     3: dict(heads=2, kv_heads=2, dim=40, vdim=8, conv=2)}),
    "top_one_every_group_kept": dict(order=(("attention", "moe"), ("delta", "moe")), experts=4, groups=(2, 2), top=1),
    "one_expert_per_group": dict(order=(("delta", "moe"),), experts=5, groups=(5, 2), top=2, shared_ff=0),
    "every_expert_chosen": dict(order=(("attention", "moe"),), experts=3, groups=None, top=3),
    "many_experts": dict(order=(("attention", "moe"), ("delta", "dense")), experts=72, groups=(8, 3), top=5, expert_ff=24),
    "long_convolution_wide_state": dict(order=(("delta", "dense"), ("delta", None)), delta=dict(heads=2, kv_heads=1, dim=136, vdim=40, conv=7)),
    "widest_delta_heads": dict(order=DELTA, delta=dict(heads=2, kv_heads=2, dim=256, vdim=72, conv=2)),
    # head sizes of the fused tensor-core attention (serving mode) with windows shorter than its 64-key tiles / longer than a page
    "fused_attention_short_window": dict(width=128, vocab=256, heads=4, kv_heads=1, dim=64, vdim=64, window=20, order=(("attention", "dense"),) * 2),
    "fused_attention_128": dict(width=128, vocab=256, heads=2, kv_heads=2, dim=128, vdim=128, window=70, softcap=3.0,
                                order=(("attention", "dense"), ("attention", None))),
    "fused_attention_causal_no_cap": dict(width=128, vocab=256, heads=6, kv_heads=2, dim=64, vdim=64, window=0, softcap=0,
                                          order=(("attention", None), ("delta", "dense"))),
    # shapes the tensor-core products take in the serving mode (steps of hundreds of tokens in the test below)
    "tensor_core_shapes": dict(width=128, vocab=256, heads=4, kv_heads=2, dim=64, vdim=64, window=96, ff=128, expert_ff=64, shared_ff=64,
                               delta=dict(heads=4, kv_heads=2, dim=64, vdim=32)),
    "packed_gated_units": dict(width=128, vocab=256, heads=4, kv_heads=2, dim=32, vdim=64, window=40, ff=256, expert_ff=128, shared_ff=128,
                               delta=dict(heads=2, kv_heads=1, dim=128, vdim=64)),
}


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_oracle(name, f32):
    cfg = ref.random_config(**CONFIGS[name])
    sd = ref.random_state_dict(cfg, seed=3)
    toks = tokens(1, 150, cfg["vocab"])  # crosses two page borders and several windows of every configuration above
    want, ok = oracle_rows(cfg, sd, toks, f32)
    with make_engine(cfg, sd, f32) as e:
        got = replay(e, toks, [len(toks)])
    check(got, want, ok, f32, least=140 if f32 or name in SERVING_ROWS else 0)


# configurations whose serving-mode comparison keeps most rows: no mixture, or mixtures in the last layer only
SERVING_ROWS = {"fused_attention_short_window", "fused_attention_128", "fused_attention_causal_no_cap", "attention_alone", "delta_alone", "dense_alone", "causal_no_window", "no_blending_and_partial_blending",
                "every_expert_chosen", "long_convolution_wide_state", "widest_delta_heads"}


@pytest.mark.parametrize("name", ["tensor_core_shapes", "packed_gated_units"])
def test_steps_of_hundreds_of_tokens_take_the_tensor_core_products(name):
    cfg = ref.random_config(**CONFIGS[name])
    sd = ref.random_state_dict(cfg, seed=5)
    toks = tokens(2, 420, cfg["vocab"])
    for f32 in (1, 0):
        want, ok = oracle_rows(cfg, sd, toks, f32)
        with make_engine(cfg, sd, f32) as e:
            check(replay(e, toks, [len(toks)]), want, ok, f32)
            check(replay(e, toks, [300, 2, 97, 2]), want, ok, f32)
    # the mixture in the last layer: a choice that flips under rounding stays in its own row, most rows count
    last = ref.random_config(**dict(CONFIGS[name], order=(("attention", "dense"), ("delta", "dense"), ("attention", "moe"))))
    sd = ref.random_state_dict(last, seed=5)
    want, ok = oracle_rows(last, sd, toks, 0)
    with make_engine(last, sd, 0) as e:
        check(replay(e, toks, [len(toks)]), want, ok, 0, least=200)
        check(replay(e, toks, [290, 2, 120]), want, ok, 0, least=200)


@pytest.mark.parametrize("f32", [1, 0])
def test_prefill_portions_and_single_tokens_agree(f32):
    cfg = ref.random_config() if f32 else ref.random_config(**CONFIGS["moe_last"])
    sd = ref.random_state_dict(cfg, seed=7)
    toks = tokens(3, 140, cfg["vocab"])
    want, ok = oracle_rows(cfg, sd, toks, f32)
    with make_engine(cfg, sd, f32) as e:
        whole = replay(e, toks, [len(toks)])
        for cuts in ([64, 64], [63, 2, 2, 61], [19, 20, 21, 2, 45], [1, 1, 1, 2, 3, 64, 5], [2, 2, 2, 3, 2], []):
            got = replay(e, toks, cuts)
            check(got, want, ok, f32, least=70)
            # the same positions, cut differently: rounding only
            assert not ok.any() or row_err(got, whole)[ok].max() < (1e-5 if f32 else 3e-2), cuts


def sharpen(cfg, factor):
    """Peaked softmax: single keys dominate, so a key wrongly seen or missed moves the logits by far more than rounding."""
    cfg = copy.deepcopy(cfg)
    for ly in cfg["layers"]:
        if ly["type"] == "attention":
            ly["mixer"]["scale"] *= factor
            ly["mixer"]["softcap"] = 40.0
    return cfg


@pytest.mark.parametrize("window", [1, 5, 63, 64, 65, 70, 130])
def test_window_edges_in_prompts_and_decoding(window):
    cfg = sharpen(ref.random_config(order=ATT * 2, window=window), 6.0)
    sd = ref.random_state_dict(cfg, seed=11)
    for p in ("l0.", "l1."):
        sd[p + "mix.sink"] = np.full_like(sd[p + "mix.sink"], -6.0)  # a weak sink: the keys carry the weight
    toks = tokens(4, 2 * window + 64 + 9, cfg["vocab"])
    want = ref.LatanexOracle(cfg, sd).forward(toks)
    # a window that is one position longer / shorter is far away
    for dw in (-1, 1):
        if window + dw < 1:
            continue
        other = ref.LatanexOracle(sharpen(ref.random_config(order=ATT * 2, window=window + dw), 6.0), sd).forward(toks)
        assert row_err(other[window:], want[window:]).max() > 50 * TOL[1]
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[1]                     # edges inside one prompt
        assert row_err(replay(e, toks, [max(1, window - 1)]), want).max() < TOL[1]            # the window fills while decoding
        assert row_err(replay(e, toks, [window + 1, 2, max(1, window - 2), 3]), want).max() < TOL[1]  # portions that start inside one
        assert row_err(replay(e, toks, [window, window]), want).max() < TOL[1]
    with make_engine(cfg, sd, 0) as e:
        assert row_err(replay(e, toks, [window + 1, 2, max(1, window - 2), 3]), want).max() < TOL[0]


@pytest.mark.parametrize("window", [5, 63, 64, 65, 130, 200])
@pytest.mark.parametrize("dim", [64, 128])
def test_window_edges_on_the_fused_attention_kernels(window, dim):
    # serving mode, head sizes of the tcgen05 kernels: windows that start inside their 64-key tiles, in prompt portions (fused
    # prefill kernel, also portions that start inside a window) and in single-token steps (TMA decode kernel)
    kw = dict(width=128, vocab=256, heads=4, kv_heads=2, dim=dim, vdim=dim, order=ATT * 2)
    cfg = sharpen(ref.random_config(window=window, **kw), 6.0)
    sd = ref.random_state_dict(cfg, seed=12)
    for p in ("l0.", "l1."):
        sd[p + "mix.sink"] = np.full_like(sd[p + "mix.sink"], -6.0)
    toks = tokens(4, 2 * window + 128 + 9, cfg["vocab"])
    want = ref.LatanexOracle(cfg, sd).forward(toks)
    for dw in (-1, 1):  # one position off is well outside the serving mode's bound
        other = ref.LatanexOracle(sharpen(ref.random_config(window=window + dw, **kw), 6.0), sd).forward(toks)
        assert row_err(other[window:], want[window:]).max() > 1.5 * TOL[0]
    with make_engine(cfg, sd, 0, ctx=640) as e:  # half the serving bound: a third of what one position off costs
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[0] / 2
        assert row_err(replay(e, toks, [window + 64, 2, 70, 64]), want).max() < TOL[0] / 2
        assert row_err(replay(e, toks, [max(1, window - 1)]), want).max() < TOL[0] / 2  # the window fills and slides while decoding


def test_single_token_steps_of_several_sequences_on_the_decode_kernel():
    cfg = ref.random_config(width=128, vocab=256, heads=6, kv_heads=2, dim=64, vdim=64, window=150,
                            order=(("attention", "dense"), ("delta", None), ("attention", None)))
    sd = ref.random_state_dict(cfg, seed=59)
    o = ref.LatanexOracle(cfg, sd)
    seqs = [tokens(70 + i, n, cfg["vocab"]) for i, n in enumerate((330, 200, 150))]
    want = [o.forward(s) for s in seqs]
    with make_engine(cfg, sd, 0, ctx=384, use_cuda_graphs=1) as e:
        ids = [e.seq_open() for _ in seqs]
        starts = (130, 3, 64)
        for i, sid in enumerate(ids):
            e.seq_step([(sid, seqs[i][:starts[i]], [])])
        got, at = [[] for _ in seqs], list(starts)
        while any(at[i] < len(seqs[i]) for i in range(3)):
            live = [i for i in range(3) if at[i] < len(seqs[i])]
            out = e.seq_step([(ids[i], [seqs[i][at[i]]], [0]) for i in live])
            for r, i in enumerate(live):
                got[i].append(out[r])
                at[i] += 1
        for i in range(3):
            assert row_err(np.stack(got[i]), want[i][starts[i]:]).max() < TOL[0]


def test_first_tokens_and_the_sink():
    cfg = ref.random_config(order=ATT, window=8)
    sd = ref.random_state_dict(cfg, seed=13)
    sd["l0.mix.sink"] = to_bf16_f32(np.linspace(0.5, 3.0, cfg["layers"][0]["mixer"]["heads"]).astype(np.float32))
    toks = tokens(5, 20, cfg["vocab"])
    want = ref.LatanexOracle(cfg, sd).forward(toks)
    without = copy.deepcopy(cfg)
    without["layers"][0]["mixer"]["sink"] = False
    bare = ref.LatanexOracle(without, sd).forward(toks)
    # the first position sees one key: without the sink its weight would be exactly one
    assert row_err(bare, want).min() > 50 * TOL[1]
    # a sink that were scaled or capped like a score would differ as well: it counts as exp(sink), once
    assert abs(ref.sink_softmax(np.array([0.3]), 2.0)[0] - 1.0 / (1.0 + np.exp(1.7))) < 1e-12
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[1]
        assert row_err(replay(e, toks, []), want).max() < TOL[1]
    with make_engine(cfg, sd, 0) as e:
        assert row_err(replay(e, toks, [3, 2]), want).max() < TOL[0]

    def no_sink(desc):
        for l in desc.layers:
            l.attn_flags &= ~ATTN_LEARNED_SINK
    sd.pop("l0.mix.sink")
    with make_engine(cfg, sd, 1, edit=no_sink) as e:  # the flag is a parameter of the mechanism
        assert row_err(replay(e, toks, [7, 2]), bare).max() < TOL[1]


def test_whole_projection_norm_cap_and_blended_values():
    # the places where a plausible other reading exists; the oracle states the design, here its alternatives must differ
    cfg = ref.random_config(order=ATT * 3, softcap=1.5)
    sd = ref.random_state_dict(cfg, seed=17)
    toks = tokens(6, 40, cfg["vocab"])
    o = ref.LatanexOracle(cfg, sd)
    want = o.forward(toks)
    m, p = cfg["layers"][0]["mixer"], o.P["layers"][0]["mix"]
    h = np.random.default_rng(1).standard_normal((5, cfg["width"]))
    q, k, v = ref.attention_qkv(h, p, m, o.eps)
    raw = (h @ p["q"].T + p["q.b"])
    assert np.allclose((q.reshape(5, -1) / p["q.norm"]) ** 2 @ np.ones(q[0].size) / q[0].size, 1.0, atol=1e-3)  # unit RMS over ALL heads
    per_head = ref.rms_unit(raw.reshape(5, m["heads"], m["dim"]), o.eps).reshape(5, -1) * p["q.norm"]
    assert np.abs(per_head - q.reshape(5, -1)).max() > 0.05
    for key, val in (("softcap", 0), ("v_mix", False)):
        alt = copy.deepcopy(cfg)
        for ly in alt["layers"]:
            ly["mixer"][key] = val
        assert row_err(ref.LatanexOracle(alt, sd).forward(toks), want).max() > 50 * TOL[1], key
    lam = dict(sd)
    lam["l0.mix.vmix"] = np.float32(0.9)  # the first blending layer's own weight is not used
    assert np.array_equal(ref.LatanexOracle(cfg, lam).forward(toks), want)
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32) as e:
            assert row_err(replay(e, toks, [33, 2]), want).max() < TOL[f32]
        with make_engine(cfg, lam, f32) as e:
            assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[f32]


def test_far_keys_and_page_borders():
    # one window of 300 positions: the last positions look back over four pages; with a peaked softmax the keys that win are
    # anywhere in it.  The same tokens under a window of 128 differ wherever a far key mattered.
    cfg = sharpen(ref.random_config(order=(("attention", "dense"),), window=300, heads=4, kv_heads=2), 8.0)
    sd = ref.random_state_dict(cfg, seed=19)
    sd["l0.mix.sink"] = np.full_like(sd["l0.mix.sink"], -8.0)
    toks = tokens(7, 290, cfg["vocab"])
    toks[-1] = toks[3]  # plant one far key: the last query finds its own key direction 286 positions back
    want = ref.LatanexOracle(cfg, sd).forward(toks)
    near = ref.LatanexOracle(sharpen(ref.random_config(order=(("attention", "dense"),), window=128, heads=4, kv_heads=2), 8.0), sd).forward(toks)
    assert row_err(near[260:], want[260:]).max() > 50 * TOL[1]
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32) as e:
            assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[f32]
            assert row_err(replay(e, toks, [255, 2, 1, 1, 1, 2]), want).max() < TOL[f32]  # decoding over the page border at 256


def slow_decay(sd, layer=0):
    """A state that forgets slowly and writes strongly: what an early token wrote is still read hundreds of tokens later."""
    sd = dict(sd)
    sd[f"l{layer}.mix.A_log"] = np.full_like(sd[f"l{layer}.mix.A_log"], -6.0)
    return sd


def test_delta_state_carries_far_tokens_convolution_tails_and_order_of_update():
    cfg = ref.random_config(order=DELTA, delta=dict(heads=4, kv_heads=2, dim=64, vdim=24, conv=4))
    sd = slow_decay(ref.random_state_dict(cfg, seed=21))
    toks = tokens(8, 140, cfg["vocab"])
    o = ref.LatanexOracle(cfg, sd)
    want = o.forward(toks)
    changed = list(toks)
    changed[2] = (changed[2] + 1) % cfg["vocab"]  # only the recurrent state can carry this to the last positions
    assert row_err(o.forward(changed)[-5:], want[-5:]).min() > 50 * TOL[1]
    # a read-out before the write (o = S_old^T q) is another model
    S = np.zeros((3, 2))
    q = k = np.array([1.0, 0.0, 0.0])
    S1, out = ref.delta_step(S, q, k, np.array([2.0, -1.0]), 0.5, 1.0)
    assert np.allclose(out, [2.0, -1.0]) and np.allclose(S1[0], [2.0, -1.0])
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32) as e:
            assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[f32]
            # portions shorter than the convolution (tails made of old and new inputs), down to single tokens
            assert row_err(replay(e, toks, [2, 2, 1, 3, 2, 64, 2, 1, 1, 2, 40]), want).max() < TOL[f32]
            assert row_err(replay(e, toks, [17]), want).max() < TOL[f32]  # 123 single-token steps


def test_long_decoding_over_windows_and_pages():
    cfg = ref.random_config(window=50)
    sd = ref.random_state_dict(cfg, seed=23)
    toks = tokens(8, 230, cfg["vocab"])
    want, ok = oracle_rows(cfg, sd, toks, 1)
    with make_engine(cfg, sd, 1) as e:
        check(replay(e, toks, [10]), want, ok, 1, least=200)  # 220 single-token steps
    dense = ref.random_config(window=50, order=(("attention", "dense"), ("delta", "dense"), ("attention", None)))
    sd = ref.random_state_dict(dense, seed=23)
    want = ref.LatanexOracle(dense, sd).forward(toks)
    with make_engine(dense, sd, 0, use_cuda_graphs=1) as e:
        assert row_err(replay(e, toks, [10]), want).max() < TOL[0]


def test_router_groups_corrections_and_weights():
    # the router alone, on inputs made for it
    cfg = ref.random_config(order=(("attention", "moe"),), experts=8, groups=(4, 2), top=3, route_scale=2.0)
    sd = ref.random_state_dict(cfg, seed=29)
    corr = np.zeros(8, np.float32)
    corr[0] = 4.0    # expert 0 alone makes group 0 one of the two kept groups and is always chosen ...
    corr[6:8] = -4.0  # ... group 3 is never kept: its corrected scores are negative, yet they must not count as zero
    sd["l0.mlp.correction"] = corr
    o = ref.LatanexOracle(cfg, sd)
    x = np.random.default_rng(0).standard_normal((64, cfg["width"]))
    r = cfg["layers"][0]["mlp"]["router"]
    idx, wt = ref.moe_route(x, o.P["layers"][0]["mlp"], r)
    assert (idx[:, 0] == 0).all() and (idx < 6).all()
    assert np.allclose(wt.sum(-1), 2.0)                       # chosen scores over their sum, times the scale
    kept = {tuple(sorted(set(i // 2 for i in row))) for row in idx}
    assert all(len(g) <= 2 for g in kept) and len(kept) > 1   # never more than the kept groups; which ones varies by token
    s, _ = ref.moe_choice_scores(x, o.P["layers"][0]["mlp"], r)
    assert np.allclose(wt, np.take_along_axis(s, idx, -1) / np.take_along_axis(s, idx, -1).sum(-1, keepdims=True) * 2.0)  # weights without correction
    toks = tokens(9, 60, cfg["vocab"])
    want = o.forward(toks)
    plain = dict(sd)
    plain["l0.mlp.correction"] = np.zeros(8, np.float32)
    assert row_err(ref.LatanexOracle(cfg, plain).forward(toks), want).max() > 50 * TOL[1]
    ungrouped = copy.deepcopy(cfg)
    del ungrouped["layers"][0]["mlp"]["router"]["groups"]
    assert row_err(ref.LatanexOracle(ungrouped, sd).forward(toks), want).max() > 50 * TOL[1]
    for f32 in (1, 0):
        _, ok = oracle_rows(cfg, sd, toks, f32)
        with make_engine(cfg, sd, f32) as e:
            check(replay(e, toks, [33, 2]), want, ok, f32)
    # negative corrected scores everywhere: the best groups are still the least negative ones
    neg = dict(sd)
    neg["l0.mlp.correction"] = to_bf16_f32(np.array([-3.0, -3.5, -2.0, -2.5, -5.0, -5.5, -4.0, -4.5], np.float32))
    idx, _ = ref.moe_route(x, ref.LatanexOracle(cfg, neg).P["layers"][0]["mlp"], r)
    assert (idx < 4).all()
    want = ref.LatanexOracle(cfg, neg).forward(toks)
    with make_engine(cfg, neg, 1) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[1]


def test_expert_clamps_and_shared_expert():
    cfg = ref.random_config(order=(("delta", "moe"),), limit=0.4, shared_limit=0.7)
    sd = ref.random_state_dict(cfg, seed=30)
    toks = tokens(10, 50, cfg["vocab"])
    want, ok = oracle_rows(cfg, sd, toks, 1)
    for key, val in (("expert", dict(ff=cfg["layers"][0]["mlp"]["expert"]["ff"], limit=40.0)), ("shared", dict(ff=48, limit=40.0)), ("shared", None)):
        alt = copy.deepcopy(cfg)
        alt["layers"][0]["mlp"][key] = val
        assert row_err(ref.LatanexOracle(alt, sd).forward(toks), want).max() > 50 * TOL[1], key  # the clamps bite, the shared unit counts
    with make_engine(cfg, sd, 1) as e:
        check(replay(e, toks, [len(toks)]), want, ok, 1, least=45)
    want, ok = oracle_rows(cfg, sd, toks, 0)
    with make_engine(cfg, sd, 0) as e:
        check(replay(e, toks, [len(toks)]), want, ok, 0)


@pytest.mark.parametrize("f32", [1, 0])
def test_mixed_batches_match_each_request_alone(f32):
    cfg = ref.random_config() if f32 else ref.random_config(**CONFIGS["moe_last"])
    sd = ref.random_state_dict(cfg, seed=31)
    seqs = [tokens(20 + i, n, cfg["vocab"]) for i, n in enumerate((150, 37, 90, 64))]
    want, oks = zip(*[oracle_rows(cfg, sd, s, f32) for s in seqs])
    plans = [[64, 2, 30, 1, 1, 1, 51], [1, 1, 1, 1, 1, 1, 31], [3, 64, 2, 1, 20], [2, 2, 2, 2, 56]]
    with make_engine(cfg, sd, f32) as e:
        solo = [replay(e, s, p) for s, p in zip(seqs, plans)]
        ids = [e.seq_open() for _ in seqs]
        at, got = [0] * 4, [[] for _ in seqs]
        plans = [list(p) for p in plans]
        step = 0
        while any(at[i] < len(seqs[i]) for i in range(4)):
            entries, who = [], []
            for i in range(4):
                if at[i] >= len(seqs[i]) or (step + i) % 5 == 4:  # every request sits out some steps
                    continue
                n = min(plans[i].pop(0) if plans[i] else 1, len(seqs[i]) - at[i])
                entries.append((ids[i], seqs[i][at[i]:at[i] + n], list(range(n))))
                who.append((i, n))
                at[i] += n
            step += 1
            if not entries:
                continue
            out, r = e.seq_step(entries), 0
            for i, n in who:
                got[i].append(out[r:r + n])
                r += n
        for sid in ids:
            e.seq_close(sid)
    for i in range(4):
        g = np.concatenate(got[i])
        check(g, want[i], oks[i], f32, least=len(seqs[i]) // 2)
        assert not oks[i].any() or row_err(g, solo[i])[oks[i]].max() < (1e-5 if f32 else 3e-2)


def test_mixed_steps_on_the_fused_attention_kernel():
    # serving mode, head size of the tcgen05 kernels: steps that carry a long portion run every entry on the fused kernel, so
    # single tokens and two-token portions of other sequences are short items of the same launch, each with its own window start
    cfg = ref.random_config(width=128, vocab=256, heads=4, kv_heads=2, dim=64, vdim=64, window=90,
                            order=(("attention", "dense"), ("delta", None), ("attention", None)))
    sd = ref.random_state_dict(cfg, seed=33)
    o = ref.LatanexOracle(cfg, sd)
    seqs = [tokens(30 + i, n, cfg["vocab"]) for i, n in enumerate((300, 140, 170))]
    want = [o.forward(s) for s in seqs]
    plans = [[100, 100, 64, 36], [1] * 3 + [70, 2, 65], [2, 2, 99, 1, 66]]
    with make_engine(cfg, sd, 0) as e:
        ids = [e.seq_open() for _ in seqs]
        at, got = [0] * 3, [[] for _ in seqs]
        while any(at[i] < len(seqs[i]) for i in range(3)):
            entries, who = [], []
            for i in range(3):
                if at[i] >= len(seqs[i]):
                    continue
                n = min(plans[i].pop(0) if plans[i] else 1, len(seqs[i]) - at[i])
                entries.append((ids[i], seqs[i][at[i]:at[i] + n], list(range(n))))
                who.append((i, n))
                at[i] += n
            out, r = e.seq_step(entries), 0
            for i, n in who:
                got[i].append(out[r:r + n])
                r += n
        for sid in ids:
            e.seq_close(sid)
    for i in range(3):
        assert row_err(np.concatenate(got[i]), want[i]).max() < TOL[0]


def test_pages_and_slots_are_reused():
    cfg = ref.random_config()
    sd = slow_decay(ref.random_state_dict(cfg, seed=37), layer=1)  # a state left behind by the slot's last owner would show
    o = ref.LatanexOracle(cfg, sd)
    with make_engine(cfg, sd, 1, max_seqs=2, ctx=192, pool=256) as e:  # 4 pages, 2 sequences
        total = e.stats()["kv_pages_total"]
        assert total == 4
        for rnd in range(4):  # every round reuses the pages and slots the previous one gave back
            a, b = tokens(40 + rnd, 130, cfg["vocab"]), tokens(50 + rnd, 60, cfg["vocab"])
            sa, sb = e.seq_open(), e.seq_open()
            with pytest.raises(hb.HBError):
                e.seq_open()
            g1 = e.seq_step([(sa, a[:100], list(range(100))), (sb, b[:33], list(range(33)))])
            g2 = e.seq_step([(sa, a[100:], list(range(30))), (sb, b[33:], list(range(27)))])
            assert e.stats()["kv_pages_free"] == 0  # 3 + 1 pages
            e.seq_close(sa)
            e.seq_close(sb)
            assert e.stats()["kv_pages_free"] == total
            wa, wb = o.forward(a), o.forward(b)
            assert row_err(np.concatenate([g1[:100], g2[:30]]), wa).max() < TOL[1]
            assert row_err(np.concatenate([g1[100:], g2[30:]]), wb).max() < TOL[1]


@pytest.mark.parametrize("f32", [1, 0])
def test_greedy_generation_through_the_scheduler(f32):
    # serving mode without routers: a choice that flips under rounding would change every later token of the sequence
    cfg = ref.random_config(vocab=200) if f32 else ref.random_config(vocab=200, order=(("attention", "dense"), ("delta", None), ("attention", "dense")))
    sd = ref.random_state_dict(cfg, seed=41)
    o = ref.LatanexOracle(cfg, sd)
    prompts = [tokens(60 + i, n, cfg["vocab"]) for i, n in enumerate((70, 5, 129))]
    with make_engine(cfg, sd, f32, max_seqs=4, ctx=256) as e:
        rids, outs = e.generate(prompts, hb.Sampling(max_tokens=24, capture=CAPTURE_STEP_LOGITS | CAPTURE_PROMPT_LOGITS))
        for p, rid, out in zip(prompts, rids, outs):
            rows = e.captured_logits(rid, CAPTURE_STEP_LOGITS)
            assert row_err(e.captured_logits(rid, CAPTURE_PROMPT_LOGITS), o.forward(p)).max() < TOL[f32]
            # teacher-forced comparison of every step's logits; ids must agree wherever the oracle's margin is clear
            st = o.new_state()
            z = o.forward(p, st)[-1]
            for k, t in enumerate(out):
                assert row_err(rows[k][None], z[None]).max() < TOL[f32]
                top2 = np.sort(z)[-2:]
                if top2[1] - top2[0] > 4 * TOL[f32] * np.sqrt((z * z).mean()):
                    assert t == int(np.argmax(z)), (k, t)
                z = o.forward([t], st)[-1]
        assert e.stats()["kv_pages_free"] == e.stats()["kv_pages_total"]


def test_continuous_batching_and_mixed_steps_match_solo_runs():
    cfg = ref.random_config(vocab=200)
    sd = ref.random_state_dict(cfg, seed=43)
    prompts = [tokens(80 + i, n, cfg["vocab"]) for i, n in enumerate((90, 17, 40, 66, 3, 120))]
    sp = hb.Sampling(max_tokens=12)
    with make_engine(cfg, sd, 1, max_seqs=4, ctx=256) as e:
        solo = [e.generate([p], sp)[1][0] for p in prompts]
        _, together = e.generate(prompts, sp)  # more prompts than slots: admission waits for finished sequences
        assert together == solo
    with make_engine(cfg, sd, 1, max_seqs=4, ctx=256, batched=128, decode_with_prefill=1, mixed_step_tokens=64) as e:
        _, mixed = e.generate(prompts, sp)  # prompts cut into 64-token portions beside the running sequences' tokens
        assert e.stats()["steps_mixed"] > 0
        assert mixed == solo
    with make_engine(cfg, sd, 1, max_seqs=4, ctx=256, use_cuda_graphs=1) as e:
        _, graphed = e.generate(prompts, sp)  # decode steps replayed from CUDA graphs (one per batch size)
        assert e.stats()["graph_launches"] > 0
        assert graphed == solo


def test_window_longer_than_the_context_and_random_weights():
    # a window no sequence can fill is causal attention: nothing may be sized by the configured number
    cfg = ref.random_config(window=1 << 20)
    sd = ref.random_state_dict(cfg, seed=47)
    toks = tokens(9, 120, cfg["vocab"])
    want, ok = oracle_rows(cfg, sd, toks, 1)
    with make_engine(cfg, sd, 1, ctx=128) as e:
        check(replay(e, toks, [70, 2, 30]), want, ok, 1, least=100)
    desc = weights_io.desc_from_hf_config(cfg)
    with hb.Engine(hb.EngineConfig(device=0, max_seqs=2, max_ctx=128, max_batched_tokens=128)) as e:
        e.load_random(desc, seed=5)
        _, outs = e.generate([tokens(1, 20, cfg["vocab"])], hb.Sampling(max_tokens=4))
        assert len(outs[0]) == 4
    desc.layers[0].kv_heads = 4  # 6 query heads do not split over 4
    with hb.Engine(hb.EngineConfig(device=0, max_seqs=2, max_ctx=128, max_batched_tokens=128)) as e:
        with pytest.raises(hb.HBError):
            e.load_random(desc, seed=5)


def test_runtime_serves_a_checkpoint_folder(tmp_path):
    import json
    from helix_b200.runtime import B200Runtime, B200RuntimeParams
    cfg = ref.random_config(vocab=200, order=(("attention", "dense"), ("delta", None), ("attention", "dense")))
    sd = ref.random_state_dict(cfg, seed=53)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    weights_io.write_safetensors(tmp_path / "model.safetensors", sd)
    rt = B200Runtime(B200RuntimeParams(model=str(tmp_path), context_length=256, serve_http=False,
                                       args=["--max-num-seqs", "4", "--max-num-batched-tokens", "256"]))
    rt.start()
    try:
        e = rt.engine
        prompt = tokens(9, 50, cfg["vocab"])
        rid = e.submit(prompt, hb.Sampling(max_tokens=8, capture=CAPTURE_STEP_LOGITS))
        out, fin = [], 0
        while not fin:
            assert e.wait(rid, 20000)
            t, fin = e.poll(rid)
            out += t
        rows = e.captured_logits(rid, CAPTURE_STEP_LOGITS)
        o = ref.LatanexOracle(cfg, sd)
        st = o.new_state()
        z = o.forward(prompt, st)[-1]
        for k, t in enumerate(out):  # teacher-forced on the engine's own ids (serving mode)
            assert row_err(rows[k][None], z[None]).max() < TOL[0]
            z = o.forward([t], st)[-1]
        assert len(out) == 8
    finally:
        rt.stop()
