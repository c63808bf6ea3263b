"""Funudra layer-list decoders through the engine (driven sequences and the scheduler) against the float64 oracle.

Every test builds its own small configuration and random bf16-representable weights (oracle/funudra_ref.py); the engine runs
them in its exact mode (fp32 weights, cache, state and products), where a lost state, a convolution input of the wrong
token, a wrong rotation or a key left out must show, and in its serving mode (bf16 weights / cache rows / GEMM operands)
with a rounding-sized bound.
"""
import copy

import numpy as np
import pytest

import helix_b200 as hb
from helix_b200 import engine as E
from helix_b200 import weights_io
from helix_b200.engine import CAPTURE_PROMPT_LOGITS, CAPTURE_STEP_LOGITS
from oracle import funudra_ref as ref
from oracle.weights import to_bf16_f32

pytestmark = pytest.mark.gpu

TOL = {1: 2e-4, 0: 6e-2}  # compute_f32 -> bound on rms(diff) / rms(expected) per logits row
M2, PAR, ATT, MEM = "mamba2", "parallel", "attention", "memory"


def row_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    return np.sqrt((d * d).mean(-1)) / np.sqrt((want * want).mean(-1))


def make_desc(cfg, sd, f32):
    """The package's reader for the design's layers; a single mixer alone ("attention" / "memory": a test's tool, not a layer
    of the design) is described by hand with the same fields."""
    real = copy.deepcopy(cfg)
    for ly in real["layers"]:
        if ly["type"] == ATT:
            ly["type"], ly["mixer"] = PAR, dict(left=ly["mixer"], right=dict(heads=1, dim=4, vdim=4, gate_cap=1.0), left_scale=1.0, right_scale=1.0)
        elif ly["type"] == MEM:
            ly["type"], ly["mixer"] = PAR, dict(left=dict(heads=1, kv_heads=1, dim=4, vdim=4, scale=1.0), right=ly["mixer"], left_scale=1.0, right_scale=1.0)
    desc = weights_io.desc_from_hf_config(real, {k: v.shape for k, v in sd.items()}, compute_f32=bool(f32))
    for i, ly in enumerate(cfg["layers"]):
        d = desc.layers[i]
        if ly["type"] == ATT:
            d.side_mixer = d.side_heads = d.side_dim = d.side_vdim = 0
            d.side_gate_cap = d.mix_scale = d.side_scale = 0.0
        elif ly["type"] == MEM:
            m = ly["mixer"]
            desc.layers[i] = E.LayerDesc(mixer=E.MIXER_MLSTM, heads=m["heads"], dim=m["dim"], vdim=m["vdim"], gate_cap=float(m["gate_cap"]),
                                         ff=d.ff, ff_kind=d.ff_kind, weights_of=d.weights_of)
    return desc


def make_engine(cfg, sd, f32, max_seqs=4, ctx=512, pool=0, batched=0, **kw):
    e = hb.Engine(hb.EngineConfig(device=0, max_seqs=max_seqs, max_ctx=ctx, max_batched_tokens=batched or ctx, kv_pool_tokens=pool, **kw))
    e.load_state_dict(make_desc(cfg, sd, f32), sd)
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


BIG = dict(width=128, vocab=256, ff=128)
CONFIGS = {
    "default": dict(),
    "mamba2_alone": dict(order=((M2, False),)),
    "parallel_alone": dict(order=((PAR, False),)),
    "attention_alone": dict(order=((ATT, False),)),
    "memory_alone": dict(order=((MEM, False),)),
    "feed_forward_everywhere": dict(order=((PAR, True), (M2, True), (ATT, True), (MEM, True))),
    "shared_tensors": dict(order=((M2, True), (PAR, True), (M2, True), (PAR, True), (M2, True)), shared={2: 0, 3: 1, 4: 0}),
    "owner_behind_its_users": dict(order=((M2, True), (PAR, True), (M2, True), (PAR, True), (M2, True)), shared={0: 2, 1: 3, 4: 2}),
    "shared_neighbours": dict(order=((PAR, False), (PAR, False), (M2, True), (M2, True)), shared={1: 0, 3: 2}),
    "one_kv_head_one_group": dict(parallel=ref.parallel_cfg(heads=4, kv_heads=1, r_heads=1), mamba2=ref.mamba2_cfg(heads=3, groups=1, norm_groups=1)),
    "no_grouping": dict(parallel=ref.parallel_cfg(heads=3, kv_heads=3), mamba2=ref.mamba2_cfg(heads=4, groups=4, norm_groups=4)),
    "five_heads_per_kv_head": dict(parallel=ref.parallel_cfg(heads=10, kv_heads=2, dim=16, vdim=8, rot_dims=16)),
    # nothing a multiple of 8 or 4: every product takes the CUDA-core GEMM, rows are loaded element by element
    "odd_sizes": dict(width=90, vocab=131, ff=50, mamba2=ref.mamba2_cfg(heads=6, vdim=5, state=7, groups=3, norm_groups=2, conv=3),
                      parallel=ref.parallel_cfg(heads=6, kv_heads=3, dim=14, vdim=10, conv=5, rot_dims=6, r_heads=5, r_dim=10, r_vdim=6)),
    # values a model may make equal or one: equal head sizes, unit weights of the mixers, no cap, unscaled rotation of the
    # whole head, single taps, one norm part
    "neutral_constants": dict(parallel=ref.parallel_cfg(dim=16, vdim=16, conv=1, rot_dims=16, factor=0, softcap=0, left_scale=1.0, right_scale=1.0,
                                                        r_dim=16, r_vdim=16), mamba2=ref.mamba2_cfg(vdim=8, state=8, conv=1, norm_groups=1)),
    "no_rotation_no_convolution": dict(order=((PAR, True), (ATT, False)), parallel=ref.parallel_cfg(rot_dims=0, conv=0)),
    "two_rotating_entries_long_taps": dict(parallel=ref.parallel_cfg(rot_dims=2, conv=7, base=7.0, factor=9.0), mamba2=ref.mamba2_cfg(conv=2)),
    "norm_parts_inside_heads": dict(order=((M2, True), (M2, False)), mamba2=ref.mamba2_cfg(heads=2, vdim=16, state=24, groups=2, norm_groups=8)),
    "wide_states": dict(order=((M2, True), (MEM, False)), mamba2=ref.mamba2_cfg(heads=2, vdim=40, state=136, groups=1, norm_groups=5),
                        parallel=ref.parallel_cfg(r_heads=2, r_dim=136, r_vdim=72)),
    "widest_states": dict(order=((MEM, False), (M2, False)), mamba2=ref.mamba2_cfg(heads=1, vdim=33, state=256, groups=1, norm_groups=3),
                          parallel=ref.parallel_cfg(r_heads=1, r_dim=256, r_vdim=34)),
    "small_states": dict(order=((M2, False), (MEM, True)), mamba2=ref.mamba2_cfg(heads=4, vdim=3, state=2, groups=2, norm_groups=1),
                         parallel=ref.parallel_cfg(r_heads=2, r_dim=3, r_vdim=1)),
    "layers_differ": dict(order=((PAR, True), (M2, False), (PAR, False), (M2, True)),
                          per_layer={2: ref.parallel_cfg(heads=2, kv_heads=1, dim=40, vdim=8, conv=2, rot_dims=40, softcap=2.0, scale=0.9, r_heads=4,
                                                         r_dim=24, r_vdim=40, gate_cap=2.5, left_scale=1.25, right_scale=0.25),
                                     3: ref.mamba2_cfg(heads=6, vdim=12, state=20, groups=3, norm_groups=4, conv=6)}),
    # head sizes of the fused tensor-core attention (serving mode)
    "fused_attention_64": dict(order=((PAR, True), (M2, False), (PAR, False)),
                               parallel=ref.parallel_cfg(heads=4, kv_heads=1, dim=64, vdim=64, rot_dims=32, r_dim=32, r_vdim=64), **BIG),
    "fused_attention_128": dict(order=((PAR, True), (ATT, False)), parallel=ref.parallel_cfg(heads=2, kv_heads=2, dim=128, vdim=128, rot_dims=128, softcap=3.0),
                                **BIG),
    # shapes the tensor-core products take in the serving mode (steps of hundreds of tokens in the test below)
    "tensor_core_shapes": dict(order=((M2, True), (PAR, True), (M2, True)), shared={2: 0}, mamba2=ref.mamba2_cfg(heads=4, vdim=32, state=64, groups=2),
                               parallel=ref.parallel_cfg(heads=4, kv_heads=2, dim=32, vdim=64, rot_dims=16, r_heads=2, r_dim=64, r_vdim=32), **BIG),
}


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_oracle(name, f32):
    cfg = ref.random_config(**CONFIGS[name])
    sd = ref.random_state_dict(cfg, seed=3)
    toks = tokens(1, 150, cfg["vocab"])  # crosses two page borders
    want = ref.FunudraOracle(cfg, sd).forward(toks)
    with make_engine(cfg, sd, f32) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[f32]
        assert row_err(replay(e, toks, [97, 2, 50]), want).max() < TOL[f32]


@pytest.mark.parametrize("name", ["tensor_core_shapes", "fused_attention_64", "fused_attention_128"])
def test_steps_of_hundreds_of_tokens_take_the_tensor_core_products(name):
    cfg = ref.random_config(**CONFIGS[name])
    sd = ref.random_state_dict(cfg, seed=5)
    toks = tokens(2, 420, cfg["vocab"])
    want = ref.FunudraOracle(cfg, sd).forward(toks)
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32) as e:
            assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[f32]
            assert row_err(replay(e, toks, [300, 2, 97, 2]), want).max() < TOL[f32]


@pytest.mark.parametrize("f32", [1, 0])
def test_prefill_portions_and_single_tokens_agree(f32):
    cfg = ref.random_config(**CONFIGS["shared_tensors"])
    sd = ref.random_state_dict(cfg, seed=7)
    toks = tokens(3, 140, cfg["vocab"])
    want = ref.FunudraOracle(cfg, sd).forward(toks)
    with make_engine(cfg, sd, f32) as e:
        whole = replay(e, toks, [len(toks)])
        for cuts in ([64, 64], [63, 2, 2, 61], [19, 20, 21, 2, 45], [1, 1, 1, 2, 3, 64, 5], [2, 2, 2, 3, 2], []):
            got = replay(e, toks, cuts)
            assert row_err(got, want).max() < TOL[f32], cuts
            assert row_err(got, whole).max() < (1e-5 if f32 else 3e-2), cuts  # the same positions, cut differently: rounding only


def test_convolution_inputs_across_portions_shorter_than_the_taps():
    # seven taps on the attention projections, six on the state-space layer: tails made of old and new inputs, and a first
    # portion shorter than the taps (zeros before the start, not the slot's last owner)
    cfg = ref.random_config(order=((PAR, False), (M2, True)), parallel=ref.parallel_cfg(conv=7), mamba2=ref.mamba2_cfg(conv=6))
    sd = ref.random_state_dict(cfg, seed=9)
    for k in list(sd):
        if k.endswith(".conv"):
            sd[k] = to_bf16_f32(sd[k] * 1.5)  # every tap counts
    toks = tokens(4, 60, cfg["vocab"])
    o = ref.FunudraOracle(cfg, sd)
    want = o.forward(toks)
    shifted = list(toks)
    shifted[10] = (shifted[10] + 1) % cfg["vocab"]
    assert row_err(o.forward(shifted)[16:17], want[16:17]).min() > 50 * TOL[1]  # the oldest tap of position 16 is position 10
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32, max_seqs=1) as e:  # one slot: every replay inherits the previous one's tails
            for cuts in ([2, 2, 1, 3, 2, 6, 7, 8, 2, 1, 1, 2], [3], [5, 1, 1, 1, 1, 1, 1, 30], [len(toks)]):
                assert row_err(replay(e, toks, cuts), want).max() < TOL[f32], cuts


def sharpen(cfg, factor):
    """Peaked softmax: single keys dominate, so a key wrongly seen or missed moves the logits by far more than rounding."""
    cfg = copy.deepcopy(cfg)
    for ly in cfg["layers"]:
        if ly["type"] == PAR:
            ly["mixer"]["left"]["scale"] *= factor
            ly["mixer"]["left"]["softcap"] = 40.0
        elif ly["type"] == ATT:
            ly["mixer"]["scale"] *= factor
            ly["mixer"]["softcap"] = 40.0
    return cfg


def near_sighted(o, toks, reach):
    """The oracle's logits if every query saw only the last `reach` keys: what losing the far keys would look like."""
    full = ref.causal_softmax_attention

    def short(q, k, v, q_pos, k_pos, scale, cap):
        out = np.zeros((q.shape[0], q.shape[1], v.shape[2]))
        for i, p in enumerate(q_pos):
            keep = (k_pos <= p) & (k_pos > p - reach)
            out[i] = full(q[i:i + 1], k[keep], v[keep], q_pos[i:i + 1], k_pos[keep], scale, cap)[0]
        return out
    ref.causal_softmax_attention = short
    try:
        return o.forward(toks)
    finally:
        ref.causal_softmax_attention = full


@pytest.mark.parametrize("name", ["attention_alone", "fused_attention_64"])
def test_far_keys_and_page_borders(name):
    # a peaked softmax puts each query's weight on a few keys anywhere in the 290 positions (four pages) behind it
    kw = dict(CONFIGS[name])
    if name == "fused_attention_64":
        kw["order"] = ((ATT, True), (ATT, False))
        kw["parallel"] = ref.parallel_cfg(heads=4, kv_heads=1, dim=64, vdim=64, rot_dims=8, base=1e6, conv=3)
    else:
        kw["parallel"] = ref.parallel_cfg(rot_dims=2, base=1e6, conv=3)
    cfg = sharpen(ref.random_config(**kw), 8.0)
    sd = ref.random_state_dict(cfg, seed=19)
    toks = tokens(7, 290, cfg["vocab"])
    o = ref.FunudraOracle(cfg, sd)
    want = o.forward(toks)
    sens = row_err(near_sighted(o, toks, 128)[200:], want[200:])  # what the keys more than two pages back are worth
    assert np.median(sens) > 3 * TOL[0]
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32) as e:
            for cuts in ([len(toks)], [255, 2, 1, 1, 1, 2], [64, 64, 128, 30]):  # whole; decoding over the page border at 256; portions that end on borders
                assert row_err(replay(e, toks, cuts), want).max() < TOL[f32], cuts


def test_rotation_at_large_positions_and_its_scaling():
    # four rotating entries with a short wavelength: positions in the hundreds turn many times
    cfg = sharpen(ref.random_config(order=((ATT, False),), parallel=ref.parallel_cfg(dim=8, rot_dims=8, base=3.0, factor=1.5, conv=0)), 3.0)
    sd = ref.random_state_dict(cfg, seed=23)
    toks = tokens(8, 400, cfg["vocab"])
    want = ref.FunudraOracle(cfg, sd).forward(toks)
    for key, val in (("factor", 1.0), ("factor", 2.0)):
        alt = copy.deepcopy(cfg)
        alt["layers"][0]["mixer"]["rot"]["scaling"][key] = val
        assert row_err(ref.FunudraOracle(alt, sd).forward(toks)[5:], want[5:]).max() > 50 * TOL[1]
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[1]
        assert row_err(replay(e, toks, [390]), want).max() < TOL[1]
    with make_engine(cfg, sd, 0) as e:
        assert row_err(replay(e, toks, [199, 2]), want).max() < TOL[0]


def remember(sd, cfg):
    """States that forget slowly: what an early token wrote is still read hundreds of tokens later."""
    sd = dict(sd)
    for k in sd:
        if k.endswith("mix.A_log"):
            sd[k] = np.full_like(sd[k], -5.0)
        if k.endswith(".f.b"):
            sd[k] = np.full_like(sd[k], 6.0)
        if k.endswith(".i.b"):
            sd[k] = np.full_like(sd[k], -1.0)
    return sd


@pytest.mark.parametrize("kind", [M2, MEM])
def test_recurrent_state_carries_far_tokens(kind):
    cfg = ref.random_config(order=((kind, True), (kind, False)))
    sd = remember(ref.random_state_dict(cfg, seed=21), cfg)
    toks = tokens(8, 200, cfg["vocab"])
    o = ref.FunudraOracle(cfg, sd)
    want = o.forward(toks)
    changed = list(toks)
    changed[2] = (changed[2] + 1) % cfg["vocab"]  # only the recurrent state can carry this to the last positions
    assert row_err(o.forward(changed)[-5:], want[-5:]).max() > 4 * TOL[1]
    # a state lost between two portions: the positions behind the cut start from nothing
    st = o.new_state()
    o.forward(toks[:120], st)
    st["layer"].clear()
    assert row_err(o.forward(toks[120:], st), want[120:]).min() > 50 * TOL[1]
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32) as e:
            assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[f32]
            assert row_err(replay(e, toks, [2, 2, 1, 3, 2, 64, 2, 1, 1, 2, 40]), want).max() < TOL[f32]
            assert row_err(replay(e, toks, [120, 2, 70]), want).max() < TOL[f32]
            assert row_err(replay(e, toks, [17]), want).max() < TOL[f32]  # 183 single-token steps


def test_first_tokens_of_a_sequence():
    # the running maximum of the gates starts at zero: with strongly negative input gates the first tokens are normalised by
    # exp(-m) = 1, not by their own weight; the convolutions see zeros before the start
    cfg = ref.random_config(order=((MEM, False), (PAR, True)), parallel=ref.parallel_cfg(gate_cap=10.0))
    sd = ref.random_state_dict(cfg, seed=25)
    for k in sd:
        if k.endswith(".i.b"):
            sd[k] = np.full_like(sd[k], -6.0)
        if k.endswith(".f.b"):
            sd[k] = np.full_like(sd[k], 3.0)
    toks = tokens(9, 12, cfg["vocab"])
    want = ref.FunudraOracle(cfg, sd).forward(toks)
    # a maximum that started at minus infinity would make the first token's output independent of the input gate's size
    m = cfg["layers"][0]["mixer"]
    q, k, v = np.ones(m["dim"]), np.ones(m["dim"]), np.ones(m["vdim"])
    o0, *_ = ref.matrix_memory_step(np.zeros((m["dim"], m["vdim"])), np.zeros(m["dim"]), 0.0, q, k, v, -6.0, -0.05)
    assert np.allclose(o0, np.exp(-6.0 + 0.05) * m["dim"] / (np.exp(0.05) + 1e-6))
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32, max_seqs=1) as e:
            assert row_err(replay(e, toks, []), want).max() < TOL[f32]       # token by token from the first
            assert row_err(replay(e, toks, [1, 2, 2]), want).max() < TOL[f32]
            assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[f32]


def test_mixer_weights_gate_cap_and_score_cap_count():
    # where a plausible other reading exists the oracle states the design; here the alternatives must differ, and the engine
    # must follow the oracle
    cfg = ref.random_config(order=((PAR, True), (PAR, False)), parallel=ref.parallel_cfg(softcap=1.5, gate_cap=1.2, left_scale=0.3, right_scale=1.7))
    sd = ref.random_state_dict(cfg, seed=27)
    toks = tokens(10, 50, cfg["vocab"])
    want = ref.FunudraOracle(cfg, sd).forward(toks)
    for path, val in ((("left", "softcap"), 0.0), (("right", "gate_cap"), 30.0), (("left_scale",), 1.0), (("right_scale",), 1.0)):
        alt = copy.deepcopy(cfg)
        for ly in alt["layers"]:
            d = ly["mixer"]
            for key in path[:-1]:
                d = d[key]
            d[path[-1]] = val
        assert row_err(ref.FunudraOracle(alt, sd).forward(toks), want).max() > 50 * TOL[1], path
    nob = {k: (np.zeros_like(v) if k.endswith("left.o.b") else v) for k, v in sd.items()}
    assert row_err(ref.FunudraOracle(cfg, nob).forward(toks), want).max() > 50 * TOL[1]  # the output bias, times the left weight
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32) as e:
            assert row_err(replay(e, toks, [33, 2]), want).max() < TOL[f32]


def test_layers_that_share_tensors_keep_their_own_state_and_cache():
    cfg = ref.random_config(order=((M2, True), (PAR, False), (M2, True), (PAR, False)), shared={2: 0, 3: 1})
    sd = remember(ref.random_state_dict(cfg, seed=29), cfg)
    toks = tokens(11, 130, cfg["vocab"])
    o = ref.FunudraOracle(cfg, sd)
    want = o.forward(toks)
    # one state for both users of a tensor set would be another model: run the oracle that way
    st, rows = o.new_state(), []
    for t in toks:
        lay = st["layer"]
        rows.append(o.forward([t], st)[0])
        lay[0], lay[1] = lay[2], lay[3]
    assert row_err(np.stack(rows)[5:], want[5:]).min() > 50 * TOL[1]
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32) as e:
            assert row_err(replay(e, toks, [70, 2, 3]), want).max() < TOL[f32]
        desc = make_desc(cfg, sd, f32)
        assert desc.layers[2].weights_of == 1 and desc.layers[3].weights_of == 2


def test_long_decoding_over_pages():
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=31)
    toks = tokens(8, 230, cfg["vocab"])
    want = ref.FunudraOracle(cfg, sd).forward(toks)
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, toks, [10]), want).max() < TOL[1]  # 220 single-token steps
    with make_engine(cfg, sd, 0, use_cuda_graphs=1) as e:
        assert row_err(replay(e, toks, [10]), want).max() < TOL[0]


def test_single_token_steps_of_several_sequences_on_the_decode_kernel():
    cfg = ref.random_config(**CONFIGS["fused_attention_64"])
    sd = ref.random_state_dict(cfg, seed=59)
    o = ref.FunudraOracle(cfg, sd)
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


@pytest.mark.parametrize("name,f32", [("shared_tensors", 1), ("shared_tensors", 0), ("fused_attention_64", 0), ("odd_sizes", 1)])
def test_mixed_batches_match_each_request_alone(name, f32):
    cfg = ref.random_config(**CONFIGS[name])
    sd = ref.random_state_dict(cfg, seed=33)
    o = ref.FunudraOracle(cfg, sd)
    seqs = [tokens(20 + i, n, cfg["vocab"]) for i, n in enumerate((150, 37, 90, 64))]
    want = [o.forward(s) for s in seqs]
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
        assert row_err(g, want[i]).max() < TOL[f32]
        assert row_err(g, solo[i]).max() < (1e-5 if f32 else 3e-2)


def test_pages_and_slots_are_reused():
    cfg = ref.random_config(order=((PAR, True), (M2, False), (PAR, False)), shared={2: 0})
    sd = remember(ref.random_state_dict(cfg, seed=37), cfg)  # a state left behind by the slot's last owner would show
    o = ref.FunudraOracle(cfg, sd)
    with make_engine(cfg, sd, 1, max_seqs=2, ctx=192, pool=256) as e:  # 4 pages, 2 sequences
        total = e.stats()["kv_pages_total"]
        assert total == 4
        for rnd in range(4):  # every pass reuses the pages and slots the previous one gave back
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
    cfg = ref.random_config(vocab=200, order=((M2, True), (PAR, True), (M2, True), (PAR, False)), shared={2: 0})
    sd = ref.random_state_dict(cfg, seed=41)
    o = ref.FunudraOracle(cfg, sd)
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


def test_second_norm_of_a_layer_without_feed_forward_is_skipped():
    cfg = ref.random_config()  # the last layer has no feed-forward
    sd = ref.random_state_dict(cfg, seed=71)
    toks = tokens(13, 40, cfg["vocab"])
    want = ref.FunudraOracle(cfg, sd).forward(toks)
    sd["l2.norm2"] = np.full(cfg["width"], 3.0, np.float32)
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[1]


def test_random_weights_and_rejected_descriptions():
    cfg = ref.random_config()
    desc = weights_io.desc_from_hf_config(cfg)
    with hb.Engine(hb.EngineConfig(device=0, max_seqs=2, max_ctx=128, max_batched_tokens=128)) as e:
        e.load_random(desc, seed=5)
        _, outs = e.generate([tokens(1, 20, cfg["vocab"])], hb.Sampling(max_tokens=4))
        assert len(outs[0]) == 4
    for edit in (lambda d: setattr(d.layers[1], "kv_heads", 3),       # 4 query heads do not split over 3
                 lambda d: setattr(d.layers[0], "norm_groups", 5),    # 32 entries do not split into 5 parts
                 lambda d: setattr(d.layers[2], "weights_of", 2),     # layer 1 is another kind of layer
                 lambda d: setattr(d.layers[1], "side_gate_cap", 0.0)):
        bad = weights_io.desc_from_hf_config(cfg)
        edit(bad)
        with hb.Engine(hb.EngineConfig(device=0, max_seqs=2, max_ctx=128, max_batched_tokens=128)) as e:
            with pytest.raises(hb.HBError):
                e.load_random(bad, seed=5)


def test_runtime_serves_a_checkpoint_folder(tmp_path):
    import json
    from helix_b200.runtime import B200Runtime, B200RuntimeParams
    cfg = ref.random_config(vocab=200, order=((M2, True), (PAR, True), (M2, False)), shared={2: 0})
    cfg["layers"][2]["mlp"] = cfg["layers"][0]["mlp"]
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
        o = ref.FunudraOracle(cfg, sd)
        st = o.new_state()
        z = o.forward(prompt, st)[-1]
        for k, t in enumerate(out):  # teacher-forced on the engine's own ids (serving mode)
            assert row_err(rows[k][None], z[None]).max() < TOL[0]
            z = o.forward([t], st)[-1]
        assert len(out) == 8
    finally:
        rt.stop()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_command(tmp_path, dtype):
    # bin/trace_run over a checkpoint folder: portions beside single tokens, requests that end and whose pages and slot the
    # next request takes, steps without wanted rows; the pool holds exactly what the live requests need (64-token pages)
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = ref.random_config(vocab=120, order=((PAR, True), (M2, True), (PAR, False), (M2, True)), shared={2: 0, 3: 1})
    sd = ref.random_state_dict(cfg, seed=61)
    model = tmp_path / "model"
    model.mkdir()
    (model / "config.json").write_text(json.dumps(cfg))
    weights_io.write_safetensors(model / "model.safetensors", sd)
    o = ref.FunudraOracle(cfg, sd)
    seqs = {k: tokens(90 + i, n, cfg["vocab"]) for i, (k, n) in enumerate((("a", 75), ("b", 40), ("c", 66), ("d", 9), ("e", 30)))}
    want = {k: o.forward(v) for k, v in seqs.items()}
    steps = [
        dict(step=0, entries=[dict(id="a", tokens=seqs["a"][:70], want=[0, 63, 64, 69])], end=[]),
        dict(step=1, entries=[dict(id="a", tokens=seqs["a"][70:71], want=[0]), dict(id="b", tokens=seqs["b"][:38], want=[])], end=[]),
        dict(step=2, entries=[dict(id="b", tokens=seqs["b"][38:], want=[1]), dict(id="a", tokens=seqs["a"][71:73], want=[0, 1]),
                              dict(id="c", tokens=seqs["c"][:2], want=[1]), dict(id="d", tokens=seqs["d"], want=[8])], end=["b", "d"]),
        dict(step=3, entries=[dict(id="c", tokens=seqs["c"][2:], want=[0, 61, 63]), dict(id="a", tokens=seqs["a"][73:], want=[1]),
                              dict(id="e", tokens=seqs["e"][:29], want=[28])], end=["a"]),
        dict(step=4, entries=[dict(id="e", tokens=seqs["e"][29:], want=[0])], end=["c", "e"]),
    ]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "320"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(5)]
    at = {k: 0 for k in seqs}
    for s in steps:
        rows = []
        for en in s["entries"]:
            rows += [want[en["id"]][at[en["id"]] + w] for w in en["want"]]
            at[en["id"]] += len(en["tokens"])
        got = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(len(rows), cfg["vocab"])
        assert row_err(got, np.stack(rows)).max() < TOL[1 if dtype == "float32" else 0], s["step"]


def test_context_longer_than_the_attention_kernels_shared_memory():
    # an engine whose context (16384 positions) is more than the per-token attention kernel can keep scores for: launches are
    # sized by the step's longest context, so sequences of ordinary length run; graph replay needs the full size and is refused
    cfg = ref.random_config(order=((PAR, True), (M2, False)))
    sd = ref.random_state_dict(cfg, seed=67)
    toks = tokens(12, 300, cfg["vocab"])
    want = ref.FunudraOracle(cfg, sd).forward(toks)
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32, ctx=16384, batched=512, pool=1024) as e:
            assert row_err(replay(e, toks, [200, 2, 90]), want).max() < TOL[f32]
    with pytest.raises(hb.HBError):
        make_engine(cfg, sd, 1, ctx=16384, batched=512, pool=1024, use_cuda_graphs=1)
