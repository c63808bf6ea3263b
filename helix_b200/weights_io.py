"""Checkpoint I/O for the runtime: safetensors -> hb_model_tensor_set, HF config.json -> ModelDesc.

The reference's backends read HF safetensors (vLLM, HF_HOME cache: api/pkg/runner/vllm_runtime.go:777-812) or GGUF
blobs (Ollama); this runtime takes the HF layout directly.  Pure stdlib + numpy: the header is JSON, tensors are
memory-mapped, bf16 payloads cross the C ABI untouched.
"""
import json
import mmap
import os
import struct

import numpy as np

from . import engine as _e
from .engine import LayerDesc, ModelDesc, StackDesc, bf16_bits, MIXER_GLA, MIXER_LATENT, MIXER_GQA, MIXER_DELTA, MIXER_MAMBA2, MIXER_MLSTM

_DT = {"BF16": (np.uint16, 2), "F16": (np.float16, 2), "F32": (np.float32, 4)}
_IGNORED = ("pooler.", "embeddings.position_ids", "rotary_emb.inv_freq", "cls.", "visual.")  # visual.: the VL tower (not served)


def read_safetensors(path):
    """Yields (name, dtype string, shape, flat numpy view over the mmap)."""
    f = open(path, "rb")
    n = struct.unpack("<Q", f.read(8))[0]
    header = json.loads(f.read(n))
    mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    base = 8 + n
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt, _ = _DT[meta["dtype"]]
        a, b = meta["data_offsets"]
        yield name, meta["dtype"], tuple(meta["shape"]), np.frombuffer(mm, dtype=dt, count=(b - a) // np.dtype(dt).itemsize, offset=base + a)


def write_safetensors(path, tensors, dtype="BF16"):
    """tensors: {name: fp32 ndarray}; stored as bf16 (or F32). Used by tests and tools."""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        a = np.ascontiguousarray(a, dtype=np.float32)
        raw = bf16_bits(a).tobytes() if dtype == "BF16" else a.tobytes()
        header[name] = {"dtype": dtype, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def canonical_name(name, arch):
    if arch == 1 and name.startswith("bert."):
        name = name[len("bert."):]
    return name


def to_bf16_bits(dtype, arr):
    if dtype == "BF16":
        return np.ascontiguousarray(arr)
    return bf16_bits(arr.astype(np.float32))


def load_safetensors(engine, desc: ModelDesc, paths):
    """Stream every tensor of the checkpoint shards into the engine's weight arena."""
    import ctypes as C
    l, h = engine._l, engine._h
    engine.load_begin(desc)
    for path in ([paths] if isinstance(paths, (str, os.PathLike)) else paths):
        for name, dt, shape, arr in read_safetensors(path):
            cname = canonical_name(name, desc.arch)
            if any(cname.startswith(p) or p in cname for p in _IGNORED):
                continue
            if getattr(desc, "tie_embeddings", 0) and cname == "lm_head.weight":
                continue
            if cname in getattr(desc, "unused_tensors", ()):
                continue
            bits = to_bf16_bits(dt, arr)
            engine._ck(l.hb_model_tensor_set(h, cname.encode(), bits.ctypes.data, bits.size))
    engine._ck(l.hb_model_load_finish(h))
    engine.desc = desc


def safetensors_shapes(paths):
    """{tensor name: shape} from the headers alone."""
    out = {}
    for path in ([paths] if isinstance(paths, (str, os.PathLike)) else paths):
        with open(path, "rb") as f:
            n = struct.unpack("<Q", f.read(8))[0]
            for name, meta in json.loads(f.read(n)).items():
                if name != "__metadata__":
                    out[name] = tuple(meta["shape"])
    return out


def risepel_desc(cfg, shapes=None, compute_f32=False):
    """config.json of a Risepel checkpoint -> StackDesc.  Every size comes from the configuration; the inner size of the
    decay projection is not a configuration key and is read from the checkpoint's tensor shapes (`l<i>.mix.a1`)."""
    layers = []
    for i, ly in enumerate(cfg["layers"]):
        m = ly["mixer"]
        mlp = ly.get("mlp")
        if mlp is not None and mlp.get("kind") != "dense":
            raise ValueError(f"layer {i}: unsupported feed-forward kind {mlp.get('kind')!r}")
        d = LayerDesc(heads=m["heads"], dim=m["dim"], vdim=m["vdim"], ff=mlp["ff"] if mlp else 0,
                      ff_limit=float(mlp["limit"]) if mlp else 0.0)
        if ly["type"] == "gla":
            d.mixer, d.tau = MIXER_GLA, float(m["tau"])
            if shapes is None or f"l{i}.mix.a1" not in shapes:
                raise ValueError(f"layer {i}: the decay rank needs the checkpoint's tensor shapes")
            d.decay_rank = int(shapes[f"l{i}.mix.a1"][0])
        elif ly["type"] == "latent_attention":
            d.mixer = MIXER_LATENT
            d.q_rank, d.kv_rank, d.rot_dim = m["q_rank"], m["kv_rank"], m["rot_dim"]
            d.rope_dims, d.rope_base = int(m["rot"]["dims"]), float(m["rot"]["base"])
            d.window, d.scale = int(m["mask"]["size"]), float(m["scale"])
            d.kv_from = int(m["kv_from"]) if m.get("kv_from") is not None else -1
        else:
            raise ValueError(f"layer {i}: unknown layer type {ly['type']!r}")
        layers.append(d)
    return StackDesc(width=cfg["width"], vocab=cfg["vocab"], layers=layers, compute_f32=int(bool(compute_f32)),
                     norm_eps=float(cfg["norm"]["eps"]), resid_alpha=float(cfg["postln_alpha"]),
                     logit_softcap=float(cfg.get("logit_softcap") or 0.0))


def lurepel_desc(cfg, shapes=None, compute_f32=False):
    """config.json of a Lurepel checkpoint -> StackDesc: grouped-query attention layers whose values are their keys, on a
    stream where each sublayer's output is normed before it is added; dense (tanh-GELU) or mixture-of-experts feed-forward.
    Every size and constant comes from the configuration."""
    layers = []
    for i, ly in enumerate(cfg["layers"]):
        if ly["type"] != "attention":
            raise ValueError(f"layer {i}: unknown layer type {ly['type']!r}")
        m = ly["mixer"]
        d = LayerDesc(mixer=MIXER_GQA, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                      scale=float(m["scale"]),
                      attn_flags=_e.ATTN_QK_UNIT_NORM | _e.ATTN_V_IS_K | _e.ATTN_UNIT_SINK | _e.ATTN_HEAD_GATE)
        mask = m.get("mask")
        if mask and mask.get("size"):
            d.mask, d.window = _e.MASK_CHUNK, int(mask["size"])
        else:
            d.mask, d.window = _e.MASK_CAUSAL, 0
        rot = m.get("rot")
        if rot and rot.get("dims"):
            d.rope_dims, d.rope_base, d.rope_pairing = int(rot["dims"]), float(rot["base"]), 1
            sc = rot.get("scaling")
            if sc:
                d.rope_factor, d.rope_low, d.rope_high = float(sc["factor"]), float(sc["low"]), float(sc["high"])
                d.rope_original = int(sc["original"])
        mlp = ly.get("mlp")
        if mlp is not None:
            kind = mlp.get("kind")
            if kind == "dense":
                d.ff_kind, d.ff = _e.FF_GELU_TANH, int(mlp["ff"])
            elif kind == "moe":
                r = mlp["router"]
                d.ff_kind, d.ff = _e.FF_MOE, int(mlp["expert"]["ff"])
                d.experts, d.identity_experts, d.top_k = int(r["experts"]), int(r.get("identity") or 0), int(r["top"])
            else:
                raise ValueError(f"layer {i}: unsupported feed-forward kind {kind!r}")
        layers.append(d)
    return StackDesc(width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=layers, compute_f32=int(bool(compute_f32)),
                     norm_eps=float(cfg["norm"]["eps"]), resid_alpha=1.0, logit_softcap=0.0, norm_place=_e.NORM_OF_OUTPUT,
                     embed_norm=1, plain_gains=1)


def latanex_desc(cfg, shapes=None, compute_f32=False):
    """config.json of a Latanex checkpoint -> StackDesc: a scaled embedding, tanh norms on both sides of every sublayer,
    windowed grouped-query attention (biased projections, whole-projection q / k norm, capped scores, learned sinks, values
    blended with the first blending layer's) and gated-delta-rule layers, silu-gated or mixture-of-experts feed-forwards
    (sigmoid router, group-limited choice, renormalised and scaled weights, clamped experts, a shared expert).  Every size
    and every constant that may differ between checkpoints comes from the configuration."""
    layers = []
    for i, ly in enumerate(cfg["layers"]):
        m = ly["mixer"]
        d = LayerDesc(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]))
        if ly["type"] == "attention":
            d.mixer, d.scale = MIXER_GQA, float(m["scale"])
            d.attn_flags = _e.ATTN_QKV_BIAS | _e.ATTN_QK_PROJ_NORM | _e.ATTN_LEARNED_SINK | (_e.ATTN_V_BLEND if m.get("v_mix") else 0)
            d.score_cap = float(m.get("softcap") or 0.0)
            mask = m.get("mask")
            if mask and mask.get("size"):
                d.mask, d.window = _e.MASK_WINDOW, int(mask["size"])
            else:
                d.mask, d.window = _e.MASK_CAUSAL, 0
        elif ly["type"] == "delta":
            d.mixer, d.conv_taps = MIXER_DELTA, int(m["conv"])
        else:
            raise ValueError(f"layer {i}: unknown layer type {ly['type']!r}")
        mlp = ly.get("mlp")
        if mlp is not None:
            kind = mlp.get("kind")
            if kind == "dense":
                d.ff_kind, d.ff = _e.FF_SILU, int(mlp["ff"])
            elif kind == "moe":
                r = mlp["router"]
                d.ff_kind, d.ff, d.ff_limit = _e.FF_MOE, int(mlp["expert"]["ff"]), float(mlp["expert"]["limit"])
                d.experts, d.top_k = int(r["experts"]), int(r["top"])
                d.router_kind, d.expert_kind, d.route_renorm = _e.ROUTER_SIGMOID, _e.EXPERT_CLAMPED, 1
                d.route_scale = float(r.get("scale", 1.0))
                g = r.get("groups")
                if g:
                    d.route_groups, d.route_keep = int(g["count"]), int(g["keep"])
                sh = mlp.get("shared")
                if sh:
                    d.shared_ff, d.shared_limit = int(sh["ff"]), float(sh["limit"])
            else:
                raise ValueError(f"layer {i}: unsupported feed-forward kind {kind!r}")
        layers.append(d)
    emb = cfg.get("embedding") or {}
    # a checkpoint may carry a blend weight for every attention layer; only layers that blend with an earlier one use theirs
    seen, unused = False, set()
    for i, d in enumerate(layers):
        if d.mixer == MIXER_GQA:
            if not (d.attn_flags & _e.ATTN_V_BLEND) or not seen:
                unused.add(f"l{i}.mix.vmix")
            seen = seen or bool(d.attn_flags & _e.ATTN_V_BLEND)
    return StackDesc(unused_tensors=frozenset(unused), width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=layers, compute_f32=int(bool(compute_f32)),
                     norm_eps=float(cfg["norm"]["eps"]), resid_alpha=1.0, logit_softcap=0.0, norm_place=_e.NORM_BOTH_SIDES,
                     norm_kind=_e.NORM_TANH, plain_gains=1, embed_scale=float(emb.get("scale", 1.0)),
                     logit_scale=float(cfg.get("logit_scale", 1.0)))


def funudra_desc(cfg, shapes=None, compute_f32=False):
    """config.json of a Funudra checkpoint -> StackDesc: a normed embedding that is also the output matrix; layers whose two
    sublayers read the same stream through two RMS norms and are added together; state-space layers with scalar decays
    ("mamba2") and layers of two mixers side by side ("parallel": grouped-query attention with convolved, biased projections,
    rotation in halves with linearly scaled frequencies, capped scores and an entry-wise output gate, beside a matrix memory
    with exponential gates); relu-squared feed-forwards; layers that use another layer's tensors.  Every size and every
    constant that may differ between checkpoints comes from the configuration."""
    layers = []
    for i, ly in enumerate(cfg["layers"]):
        m = ly["mixer"]
        if ly["type"] == "mamba2":
            d = LayerDesc(mixer=MIXER_MAMBA2, heads=int(m["heads"]), vdim=int(m["vdim"]), dim=int(m["state"]), kv_heads=int(m["groups"]),
                          norm_groups=int(m.get("norm_groups") or 1), conv_taps=int(m.get("conv") or 1))
        elif ly["type"] == "parallel":
            l, r = m["left"], m["right"]
            d = LayerDesc(mixer=MIXER_GQA, heads=int(l["heads"]), kv_heads=int(l["kv_heads"]), dim=int(l["dim"]), vdim=int(l["vdim"]),
                          scale=float(l["scale"]), score_cap=float(l.get("softcap") or 0.0), mask=_e.MASK_CAUSAL, window=0,
                          attn_flags=_e.ATTN_QKV_BIAS | _e.ATTN_OUT_GATE | _e.ATTN_OUT_BIAS)
            if l.get("conv"):
                d.attn_flags |= _e.ATTN_QKV_CONV
                d.conv_taps = int(l["conv"])
            rot = l.get("rot")
            if rot and rot.get("dims"):
                d.rope_dims, d.rope_base, d.rope_pairing = int(rot["dims"]), float(rot["base"]), 0
                sc = rot.get("scaling")
                if sc and sc.get("factor"):
                    d.rope_linear = float(sc["factor"])
            d.side_mixer, d.side_heads, d.side_dim, d.side_vdim = MIXER_MLSTM, int(r["heads"]), int(r["dim"]), int(r["vdim"])
            d.side_gate_cap = float(r["gate_cap"])
            d.mix_scale, d.side_scale = float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0))
            if d.mix_scale == 0.0 or d.side_scale == 0.0:
                raise ValueError(f"layer {i}: a mixer weight of zero is not representable (0 means 1)")
        else:
            raise ValueError(f"layer {i}: unknown layer type {ly['type']!r}")
        mlp = ly.get("mlp")
        if mlp is not None:
            if mlp.get("kind") != "dense":
                raise ValueError(f"layer {i}: unsupported feed-forward kind {mlp.get('kind')!r}")
            d.ff_kind, d.ff = _e.FF_RELU2, int(mlp["ff"])
        if ly.get("weights_of") is not None:
            j, seen = int(ly["weights_of"]), {i}
            while cfg["layers"][j].get("weights_of") is not None:  # a layer that itself borrows: follow to the tensors' owner
                if j in seen:
                    raise ValueError(f"layer {i}: weights_of runs in a circle")
                seen.add(j)
                j = int(cfg["layers"][j]["weights_of"])
            if j == i:
                raise ValueError(f"layer {i}: weights_of names the layer itself")
            d.weights_of = j + 1
        layers.append(d)
    # a checkpoint may carry the second norm of a layer that has no feed-forward to read it
    unused = frozenset(f"l{i}.norm2" for i, d in enumerate(layers) if d.ff == 0)
    return StackDesc(unused_tensors=unused, width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=layers, compute_f32=int(bool(compute_f32)),
                     norm_eps=float(cfg["norm"]["eps"]), resid_alpha=1.0, logit_softcap=0.0, norm_place=_e.NORM_PARALLEL,
                     embed_norm=1, plain_gains=1, tie_head=1)


# layer-list decoders by config.json "architecture"
STACK_READERS = {"Risepel": risepel_desc, "Lurepel": lurepel_desc, "Latanex": latanex_desc, "Funudra": funudra_desc}


def desc_from_hf_config(cfg, shapes=None, compute_f32=False):
    """config.json (dict or path) -> ModelDesc (Llama- and Qwen2-family decoders, BERT-family encoders) or StackDesc
    (layer-list decoders: "architecture" names one of STACK_READERS; `shapes` = safetensors_shapes of the checkpoint)."""
    if not isinstance(cfg, dict):
        with open(cfg) as f:
            cfg = json.load(f)
    if cfg.get("architecture") in STACK_READERS:
        return STACK_READERS[cfg["architecture"]](cfg, shapes, compute_f32)
    if compute_f32:
        raise ValueError("fp32 compute exists for layer-list decoders only")
    mt = cfg.get("model_type", "")
    if mt in ("qwen2", "qwen2_vl") and "text_config" in cfg:  # VL checkpoints nest the language model's configuration
        cfg = dict(cfg["text_config"], model_type="qwen2")
        mt = "qwen2"
    if mt in ("llama", "qwen2"):
        heads = cfg["num_attention_heads"]
        rope = cfg.get("rope_parameters") or cfg.get("rope_scaling") or {}
        d = ModelDesc(arch=0, hidden=cfg["hidden_size"], layers=cfg["num_hidden_layers"], heads=heads,
                      kv_heads=cfg.get("num_key_value_heads", heads), head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
                      ffn=cfg["intermediate_size"], vocab=cfg["vocab_size"], max_pos=cfg.get("max_position_embeddings", 8192),
                      tie_embeddings=int(bool(cfg.get("tie_word_embeddings", False))), norm_eps=cfg.get("rms_norm_eps", 1e-5),
                      rope_theta=float(rope.get("rope_theta", cfg.get("rope_theta", 10000.0))),
                      qkv_bias=int(mt == "qwen2"))  # Qwen2: biases on q/k/v, otherwise the Llama layer
        if (rope.get("rope_type") or rope.get("type")) == "llama3":
            d.rope_factor = float(rope["factor"])
            d.rope_low_freq_factor = float(rope["low_freq_factor"])
            d.rope_high_freq_factor = float(rope["high_freq_factor"])
            d.rope_orig_max_pos = int(rope["original_max_position_embeddings"])
        return d
    if mt == "bert":
        heads = cfg["num_attention_heads"]
        return ModelDesc(arch=1, hidden=cfg["hidden_size"], layers=cfg["num_hidden_layers"], heads=heads, kv_heads=heads,
                         head_dim=cfg["hidden_size"] // heads, ffn=cfg["intermediate_size"], vocab=cfg["vocab_size"],
                         max_pos=cfg["max_position_embeddings"], type_vocab=cfg.get("type_vocab_size", 2),
                         norm_eps=cfg.get("layer_norm_eps", 1e-12))
    raise ValueError(f"unsupported model_type {mt!r}")
