"""Host-side binding of the engine C ABI (include/helix_b200.h).

Mirrors, one to one, what the Go ``B200Runtime`` shim does over cgo: create an engine
for a slot's ``gpu_index`` / ``model_memory_requirement``, load a model, start the step loop, then
submit / poll token ids (chat) or call ``embed`` (RAG ingest).
"""
import ctypes as C
from dataclasses import dataclass, field, asdict

import numpy as np

from . import _lib
from ._lib import EngineCfg, LayerDescC, ModelDescC, SamplingC, SeqFeedC, StackDescC, StatsC

CAPTURE_STEP_LOGITS = 1
CAPTURE_PROMPT_LOGITS = 2


class HBError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"hb error {code}: {msg}")
        self.code = code


@dataclass
class EngineConfig:
    device: int = 0
    memory_budget_bytes: int = 0
    max_seqs: int = 256
    max_ctx: int = 8192
    max_batched_tokens: int = 16384
    kv_page_size: int = 64
    use_cuda_graphs: int = 0
    enable_prefix_cache: int = 0
    sm_budget: int = 0            # SMs this engine's persistent kernels may occupy (0 = all): multi-model packing
    sm_partition: int = 0         # 1: enforce sm_budget with a CUDA green context
    stream_priority: int = 0      # 1: high-priority stream
    decode_with_prefill: int = 0  # 1: running sequences decode inside prefill steps (mixed batches)
    fused_decode: int = 0         # 1: decode GEMMs with tile finishers instead of separate row kernels (measured slower)
    mixed_step_tokens: int = 0    # token budget of a step that carries decode rows (0 = 2048)
    kv_pool_tokens: int = 0       # cap of the cache pool in tokens (0 = max_seqs full contexts)

    def to_c(self):
        return EngineCfg(self.device, self.memory_budget_bytes, self.max_seqs, self.max_ctx, self.max_batched_tokens,
                         self.kv_page_size, self.use_cuda_graphs, self.enable_prefix_cache, self.sm_budget,
                         self.sm_partition, self.stream_priority, self.decode_with_prefill, self.fused_decode, self.mixed_step_tokens,
                         self.kv_pool_tokens)


@dataclass
class ModelDesc:
    arch: int = 0
    hidden: int = 0
    layers: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    ffn: int = 0
    vocab: int = 0
    max_pos: int = 0
    type_vocab: int = 0
    tie_embeddings: int = 0
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_factor: float = 0.0
    rope_low_freq_factor: float = 1.0
    rope_high_freq_factor: float = 4.0
    rope_orig_max_pos: int = 0
    qkv_bias: int = 0     # Qwen2-family decoders: biases on the q/k/v projections

    def to_c(self):
        return ModelDescC(self.arch, self.hidden, self.layers, self.heads, self.kv_heads, self.head_dim, self.ffn,
                          self.vocab, self.max_pos, self.type_vocab, self.tie_embeddings, self.norm_eps,
                          self.rope_theta, self.rope_factor, self.rope_low_freq_factor, self.rope_high_freq_factor,
                          self.rope_orig_max_pos, self.qkv_bias)


MIXER_GLA = 0
MIXER_LATENT = 1
MIXER_GQA = 2
MIXER_DELTA = 3
MIXER_MAMBA2 = 4
MIXER_MLSTM = 5
MASK_WINDOW, MASK_CHUNK, MASK_CAUSAL = 0, 1, 2
FF_CLAMPED, FF_GELU_TANH, FF_MOE, FF_SILU, FF_RELU2 = 0, 1, 2, 3, 4
NORM_OF_SUM, NORM_OF_OUTPUT, NORM_BOTH_SIDES, NORM_PARALLEL = 0, 1, 2, 3
NORM_RMS, NORM_TANH = 0, 1
ROUTER_SOFTMAX, ROUTER_SIGMOID = 0, 1
EXPERT_SILU, EXPERT_CLAMPED = 0, 1
ATTN_QK_UNIT_NORM, ATTN_V_IS_K, ATTN_UNIT_SINK, ATTN_HEAD_GATE = 1, 2, 4, 8
ATTN_QKV_BIAS, ATTN_QK_PROJ_NORM, ATTN_LEARNED_SINK, ATTN_V_BLEND = 16, 32, 64, 128
ATTN_QKV_CONV, ATTN_OUT_GATE, ATTN_OUT_BIAS = 256, 512, 1024


@dataclass
class LayerDesc:
    """One layer of a layer-list decoder (hb_layer_desc)."""
    mixer: int = MIXER_GLA
    heads: int = 0
    dim: int = 0
    vdim: int = 0
    tau: float = 1.0
    decay_rank: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    rot_dim: int = 0
    rope_dims: int = 0
    window: int = 0
    kv_from: int = -1
    rope_base: float = 10000.0
    scale: float = 1.0
    ff: int = 0
    ff_limit: float = 0.0
    kv_heads: int = 0          # GQA
    mask: int = MASK_WINDOW
    attn_flags: int = 0
    rope_pairing: int = 0      # 1: interleaved pairs (2i, 2i+1)
    rope_factor: float = 0.0   # <= 0: no frequency scaling
    rope_low: float = 1.0
    rope_high: float = 4.0
    rope_original: int = 0
    ff_kind: int = FF_CLAMPED
    experts: int = 0           # FF_MOE: experts with weights (ff = inner size of one)
    identity_experts: int = 0
    top_k: int = 0
    score_cap: float = 0.0     # GQA: cap * tanh(s / cap) on the scaled scores; <= 0: off
    conv_taps: int = 0         # DELTA
    router_kind: int = ROUTER_SOFTMAX
    route_groups: int = 0      # FF_MOE: groups of neighbouring experts / groups that stay eligible
    route_keep: int = 0
    route_renorm: int = 0      # 1: chosen scores divided by their sum
    route_scale: float = 0.0   # 0 = 1
    expert_kind: int = EXPERT_SILU
    shared_ff: int = 0         # FF_MOE: a unit every token uses
    shared_limit: float = 0.0
    weights_of: int = 0        # j + 1: the layer uses layer j's tensors (cache and state stay its own); 0: its own
    rope_linear: float = 0.0   # GQA: rotation frequencies divided by it; <= 0: off
    norm_groups: int = 0       # MAMBA2: equal parts of the gated output normed separately
    gate_cap: float = 0.0      # MLSTM
    side_mixer: int = 0        # a second mixer beside the first when side_heads > 0 (MIXER_MLSTM)
    side_heads: int = 0
    side_dim: int = 0
    side_vdim: int = 0
    side_gate_cap: float = 0.0
    mix_scale: float = 0.0     # weights of the two mixers' outputs; 0 = 1
    side_scale: float = 0.0

    def to_c(self):
        return LayerDescC(self.mixer, self.heads, self.dim, self.vdim, self.tau, self.decay_rank, self.q_rank, self.kv_rank,
                          self.rot_dim, self.rope_dims, self.window, self.kv_from, self.rope_base, self.scale, self.ff, self.ff_limit,
                          self.kv_heads, self.mask, self.attn_flags, self.rope_pairing, self.rope_factor, self.rope_low,
                          self.rope_high, self.rope_original, self.ff_kind, self.experts, self.identity_experts, self.top_k,
                          self.score_cap, self.conv_taps, self.router_kind, self.route_groups, self.route_keep, self.route_renorm,
                          self.route_scale, self.expert_kind, self.shared_ff, self.shared_limit, self.weights_of, self.rope_linear,
                          self.norm_groups, self.gate_cap, self.side_mixer, self.side_heads, self.side_dim, self.side_vdim,
                          self.side_gate_cap, self.mix_scale, self.side_scale)


@dataclass
class StackDesc:
    """A layer-list decoder (hb_stack_desc + hb_layer_desc[]): arch 2."""
    width: int = 0
    vocab: int = 0
    layers: list = field(default_factory=list)
    compute_f32: int = 0
    norm_eps: float = 1e-6
    resid_alpha: float = 1.0
    logit_softcap: float = 0.0
    norm_place: int = NORM_OF_SUM
    embed_norm: int = 0
    plain_gains: int = 0
    norm_kind: int = NORM_RMS
    embed_scale: float = 0.0   # 0 = 1
    logit_scale: float = 0.0   # 0 = 1
    tie_head: int = 0          # 1: logits from the embedding table
    arch: int = 2
    unused_tensors: frozenset = frozenset()  # checkpoint tensors the design names but this stack has no use for (skipped at load)

    @property
    def hidden(self):
        return self.width

    @property
    def max_pos(self):
        return 1 << 20  # rotary angles and the recurrence are computed per position: no trained position limit

    def to_c(self):
        arr = (LayerDescC * len(self.layers))(*[l.to_c() for l in self.layers])
        return StackDescC(self.width, self.vocab, len(self.layers), self.compute_f32, self.norm_eps, self.resid_alpha,
                          self.logit_softcap, self.norm_place, self.embed_norm, self.plain_gains, self.norm_kind, self.embed_scale,
                          self.logit_scale, self.tie_head), arr


@dataclass
class Sampling:
    temperature: float = 0.0
    seed: int = 0
    max_tokens: int = 16
    eos_token: int = -1
    capture: int = 0
    top_k: int = 0      # <= 0: off
    top_p: float = 1.0  # outside (0, 1): off
    logprobs: int = 0   # n >= 1: chosen token + the n-1 most likely alternatives per generated token (n <= 21)
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0

    def to_c(self):
        return SamplingC(self.temperature, self.seed, self.max_tokens, self.eos_token, self.capture, self.top_k, self.top_p,
                         self.logprobs, self.presence_penalty, self.frequency_penalty)


def bf16_bits(a):
    """fp32 ndarray -> uint16 bf16 bit patterns (round to nearest even) — how weights cross the C ABI."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def replica_unique_id() -> bytes:
    """ncclGetUniqueId through the library (hb_replica_unique_id): 128 bytes to hand to every replica."""
    buf = C.create_string_buffer(128)
    rc = _lib.lib().hb_replica_unique_id(buf)
    if rc != 0:
        raise HBError(rc, "hb_replica_unique_id failed (libnccl.so.2 not available?)")
    return buf.raw


def gguf_describe(path) -> ModelDesc:
    d = ModelDescC()
    rc = _lib.lib().hb_gguf_describe(str(path).encode(), C.byref(d))
    if rc != 0:
        raise HBError(rc, (_lib.lib().hb_last_error(None) or b"").decode())
    return ModelDesc(**{k: getattr(d, k) for k, _ in ModelDescC._fields_ if not k.startswith("reserved")})


def gguf_read_tensor(path, hf_name):
    """One tensor of a GGUF file as fp32 [rows, cols] in the HF layout (dequantised, q/k rows un-permuted)."""
    l = _lib.lib()
    rows, cols = C.c_size_t(), C.c_size_t()
    rc = l.hb_gguf_read_tensor(str(path).encode(), hf_name.encode(), None, 0, C.byref(rows), C.byref(cols))
    if rc not in (0, -6):
        raise HBError(rc, (l.hb_last_error(None) or b"").decode() or f"tensor {hf_name} not in {path}")
    out = np.empty((rows.value, cols.value), np.float32)
    rc = l.hb_gguf_read_tensor(str(path).encode(), hf_name.encode(), out.ctypes.data, out.size, C.byref(rows), C.byref(cols))
    if rc != 0:
        raise HBError(rc, "hb_gguf_read_tensor failed")
    return out


def memory_estimate(desc: ModelDesc, cfg: EngineConfig):
    l = _lib.lib()
    w, kv, ws = C.c_uint64(), C.c_uint64(), C.c_uint64()
    rc = l.hb_memory_estimate(C.byref(desc.to_c()), C.byref(cfg.to_c()), C.byref(w), C.byref(kv), C.byref(ws))
    if rc != 0:
        raise HBError(rc, "hb_memory_estimate: unsupported description")
    return {"weights": w.value, "kv": kv.value, "workspace": ws.value}


class Engine:
    def __init__(self, cfg: EngineConfig):
        self._l = _lib.lib()
        self._h = C.c_void_p()
        self.cfg = cfg
        ccfg = cfg.to_c()
        rc = self._l.hb_engine_create(C.byref(ccfg), C.byref(self._h))
        if rc != 0:
            raise HBError(rc, (self._l.hb_last_error(None) or b"").decode())
        self.desc = None

    def _ck(self, rc):
        if rc != 0:
            raise HBError(rc, (self._l.hb_last_error(self._h) or b"").decode())

    def close(self):
        if self._h:
            self._l.hb_engine_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # ---- model load
    def load_random(self, desc, seed=0):
        if isinstance(desc, StackDesc):
            sd, layers = desc.to_c()
            self._ck(self._l.hb_model_load_random_stack(self._h, C.byref(sd), layers, seed))
        else:
            self._ck(self._l.hb_model_load_random(self._h, C.byref(desc.to_c()), seed))
        self.desc = desc

    def load_begin(self, desc):
        if isinstance(desc, StackDesc):
            sd, layers = desc.to_c()
            self._ck(self._l.hb_model_load_begin_stack(self._h, C.byref(sd), layers))
        else:
            self._ck(self._l.hb_model_load_begin(self._h, C.byref(desc.to_c())))

    def load_state_dict(self, desc, tensors):
        """tensors: {HF checkpoint name: fp32/bf16-representable ndarray}."""
        self.load_begin(desc)
        for name, a in tensors.items():
            if name in getattr(desc, "unused_tensors", ()):
                continue
            bits = bf16_bits(a)
            self._ck(self._l.hb_model_tensor_set(self._h, name.encode(), bits.ctypes.data, bits.size))
        self._ck(self._l.hb_model_load_finish(self._h))
        self.desc = desc

    def load_gguf(self, path):
        """A llama.cpp / Ollama GGUF blob: description from its metadata, tensors dequantised to bf16 (hb_model_load_gguf)."""
        self.desc = gguf_describe(path)
        self._ck(self._l.hb_model_load_gguf(self._h, str(path).encode()))

    def load_broadcast(self, desc: ModelDesc, uid: bytes, rank: int, world: int):
        """Replica load (hb_model_load_broadcast): rank 0 sends its loaded arena, the others receive it. Returns seconds."""
        sec = C.c_double()
        buf = C.create_string_buffer(bytes(uid), 128)
        self._ck(self._l.hb_model_load_broadcast(self._h, C.byref(desc.to_c()), buf, rank, world, C.byref(sec)))
        self.desc = desc
        return sec.value

    def weights_arena(self):
        p, n = C.c_void_p(), C.c_size_t()
        self._ck(self._l.hb_model_weights_arena(self._h, C.byref(p), C.byref(n)))
        return p.value, n.value

    # ---- generation
    def start(self):
        self._ck(self._l.hb_engine_start(self._h))

    def stop(self):
        self._ck(self._l.hb_engine_stop(self._h))

    def set_mixed(self, on, tokens=0):
        """decode_with_prefill / mixed_step_tokens of a live engine (next step on)."""
        self._ck(self._l.hb_engine_set_mixed(self._h, int(bool(on)), int(tokens)))

    def step(self):
        did = C.c_int()
        self._ck(self._l.hb_step(self._h, C.byref(did)))
        return bool(did.value)

    def submit(self, tokens, sampling: Sampling):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        rid = C.c_uint64()
        sp = sampling.to_c()
        self._ck(self._l.hb_submit(self._h, t.ctypes.data, t.size, C.byref(sp), C.byref(rid)))
        return rid.value

    def poll(self, rid, cap=4096):
        buf = np.empty(cap, dtype=np.int32)
        n, fin = C.c_int32(), C.c_int32()
        self._ck(self._l.hb_poll(self._h, rid, buf.ctypes.data, cap, C.byref(n), C.byref(fin)))
        return buf[:n.value].tolist(), fin.value

    def wait(self, rid, timeout_ms=-1):
        return self._l.hb_wait(self._h, rid, timeout_ms) == 0

    def cancel(self, rid):
        self._ck(self._l.hb_cancel(self._h, rid))

    def release(self, rid):
        self._ck(self._l.hb_release(self._h, rid))

    def captured_logits(self, rid, which):
        rows = C.c_int32()
        self._ck(self._l.hb_captured_logits(self._h, rid, which, None, 0, C.byref(rows)))
        out = np.empty((rows.value, self.desc.vocab), dtype=np.float32)
        if rows.value:
            self._ck(self._l.hb_captured_logits(self._h, rid, which, out.ctypes.data, out.size, C.byref(rows)))
        return out

    def logprobs(self, rid, first_row=0, max_rows=4096):
        """(ids [rows, width], logprobs [rows, width]): column 0 = the sampled token, then the most likely tokens."""
        rows, width = C.c_int32(), C.c_int32()
        self._ck(self._l.hb_logprobs(self._h, rid, first_row, 0, None, None, C.byref(rows), C.byref(width)))
        w = max(1, width.value)
        ids = np.empty((max_rows, w), dtype=np.int32)
        lps = np.empty((max_rows, w), dtype=np.float32)
        self._ck(self._l.hb_logprobs(self._h, rid, first_row, max_rows, ids.ctypes.data, lps.ctypes.data, C.byref(rows),
                                     C.byref(width)))
        return ids[:rows.value], lps[:rows.value]

    def generate(self, prompts, sampling: Sampling):
        """Synchronous helper: drive hb_step on this thread until every prompt finished."""
        rids = [self.submit(p, sampling) for p in prompts]
        outs = [[] for _ in rids]
        done = [False] * len(rids)
        while not all(done):
            self.step()
            for i, r in enumerate(rids):
                if not done[i]:
                    toks, fin = self.poll(r)
                    outs[i] += toks
                    done[i] = fin != 0
        return rids, outs

    # ---- driven sequences: the caller feeds token ids, nothing is sampled (hb_seq_*)
    def seq_open(self):
        sid = C.c_uint64()
        self._ck(self._l.hb_seq_open(self._h, C.byref(sid)))
        return sid.value

    def seq_close(self, sid):
        self._ck(self._l.hb_seq_close(self._h, sid))

    def seq_step(self, entries):
        """entries: [(seq id, tokens, want positions)] -> fp32 [sum(len(want)), vocab]; ONE engine step over all entries."""
        keep, arr = [], (SeqFeedC * len(entries))()
        rows = 0
        for i, (sid, toks, want) in enumerate(entries):
            t = np.ascontiguousarray(toks, dtype=np.int32)
            w = np.ascontiguousarray(want, dtype=np.int32)
            keep += [t, w]
            arr[i] = SeqFeedC(sid, t.ctypes.data, t.size, w.ctypes.data if w.size else None, w.size)
            rows += w.size
        out = np.empty((rows, self.desc.vocab), dtype=np.float32)
        got = C.c_int32()
        self._ck(self._l.hb_seq_step(self._h, arr, len(entries), out.ctypes.data if rows else None, out.size, C.byref(got)))
        return out

    # ---- embeddings
    def embed(self, seqs):
        lens = [len(s) for s in seqs]
        offsets = np.zeros(len(seqs) + 1, dtype=np.int32)
        offsets[1:] = np.cumsum(lens)
        toks = np.concatenate([np.asarray(s, dtype=np.int32) for s in seqs]) if seqs else np.zeros(0, np.int32)
        return self.embed_flat(toks, offsets)

    def embed_flat(self, tokens, offsets, out=None):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        offsets = np.ascontiguousarray(offsets, dtype=np.int32)
        n = offsets.size - 1
        if out is None:
            out = np.empty((n, self.desc.hidden), dtype=np.float32)
        self._ck(self._l.hb_embed(self._h, tokens.ctypes.data, offsets.ctypes.data, n, out.ctypes.data))
        return out

    def stats(self):
        s = StatsC()
        self._ck(self._l.hb_get_stats(self._h, C.byref(s)))
        out = {}
        for k, _ in StatsC._fields_:
            if k.startswith("reserved"):
                continue
            v = getattr(s, k)
            out[k] = list(v) if hasattr(v, "__len__") else v
        return out

    def set_profile(self, on):
        self._ck(self._l.hb_set_profile(self._h, int(bool(on))))
