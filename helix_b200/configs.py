"""Model shapes named by BASELINE.json / SURVEY.md §8a (random-init; no checkpoints offline)."""
from .engine import ModelDesc

LLAMA = 0
BERT = 1
RISEPEL = 2  # layer-list decoders (engine.StackDesc)


def llama3_8b():
    return ModelDesc(arch=LLAMA, hidden=4096, layers=32, heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256,
                     max_pos=8192, tie_embeddings=0, norm_eps=1e-5, rope_theta=500000.0)


def llama32_1b():
    return ModelDesc(arch=LLAMA, hidden=2048, layers=16, heads=32, kv_heads=8, head_dim=64, ffn=8192, vocab=128256,
                     max_pos=131072, tie_embeddings=1, norm_eps=1e-5, rope_theta=500000.0, rope_factor=32.0,
                     rope_low_freq_factor=1.0, rope_high_freq_factor=4.0, rope_orig_max_pos=8192)


def bge_base():
    return ModelDesc(arch=BERT, hidden=768, layers=12, heads=12, kv_heads=12, head_dim=64, ffn=3072, vocab=30522,
                     max_pos=512, type_vocab=2, norm_eps=1e-12)


def tiny_llama(layers=2, head_dim=64, vocab=1000, rope_scaling=False):
    heads, kv = 4, 2
    return ModelDesc(arch=LLAMA, hidden=heads * head_dim, layers=layers, heads=heads, kv_heads=kv, head_dim=head_dim,
                     ffn=512, vocab=vocab, max_pos=4096, tie_embeddings=0, norm_eps=1e-5, rope_theta=500000.0,
                     rope_factor=32.0 if rope_scaling else 0.0, rope_low_freq_factor=1.0, rope_high_freq_factor=4.0,
                     rope_orig_max_pos=256 if rope_scaling else 0)


def dse_qwen2_2b():
    """Text backbone shape of MrLight/dse-qwen2-2b-mrl-v1 (Qwen2-VL-2B), the reference's default embedding model served
    with `--task embed` (api/pkg/model/models.go:421-433): q/k/v biases, GQA 12/2, tied embeddings, last-token pooling."""
    return ModelDesc(arch=LLAMA, hidden=1536, layers=28, heads=12, kv_heads=2, head_dim=128, ffn=8960, vocab=151936,
                     max_pos=32768, tie_embeddings=1, norm_eps=1e-6, rope_theta=1000000.0, qkv_bias=1)


def tiny_qwen2(layers=2, vocab=1000):
    """Qwen2-style decoder in miniature: q/k/v biases, GQA group 6 (12 q heads over 2 kv heads), tied embeddings."""
    return ModelDesc(arch=LLAMA, hidden=768, layers=layers, heads=12, kv_heads=2, head_dim=64, ffn=512, vocab=vocab,
                     max_pos=4096, tie_embeddings=1, norm_eps=1e-6, rope_theta=1000000.0, qkv_bias=1)


def tiny_bert(layers=2, vocab=1000):
    return ModelDesc(arch=BERT, hidden=256, layers=layers, heads=4, kv_heads=4, head_dim=64, ffn=512, vocab=vocab,
                     max_pos=512, type_vocab=2, norm_eps=1e-12)


def risepel_stack(width, layers, ff=None, window=512, pattern=("gla", "latent", "gla", "gla"), vocab=32768, compute_f32=False):
    """A Risepel-design stack at sizes that resemble a served model's layers (random-init benchmarks): per width, heads of
    128 value channels; GLA layers with 64 key channels per head and a rank-64 decay projection; latent-attention layers with
    a 512-wide cache latent, 64 rotary dims, queries through a width/4 latent, a sliding window and a feed-forward after
    every attention layer; one layer in four is attention, every second attention layer reads the cache rows of the one
    before it."""
    from .engine import LayerDesc, StackDesc, MIXER_GLA, MIXER_LATENT
    heads = max(1, width // 128)
    ff = ff or (width * 4)
    out, lat_seen, last_own = [], 0, -1
    for i in range(layers):
        kind = pattern[i % len(pattern)]
        if kind == "gla":
            out.append(LayerDesc(mixer=MIXER_GLA, heads=heads, dim=64, vdim=128, tau=16.0, decay_rank=64))
        else:
            share = lat_seen % 2 == 1
            out.append(LayerDesc(mixer=MIXER_LATENT, heads=heads, dim=128, vdim=128, q_rank=max(64, width // 4), kv_rank=512,
                                 rot_dim=64, rope_dims=64, window=window, kv_from=last_own if share else -1, rope_base=1e6,
                                 scale=(128 + 64) ** -0.5, ff=ff, ff_limit=7.0))
            if not share:
                last_own = i
            lat_seen += 1
    return StackDesc(width=width, vocab=vocab, layers=out, compute_f32=int(compute_f32), norm_eps=1e-6, resid_alpha=2.0,
                     logit_softcap=30.0)


def lurepel_stack(width, layers, ff=None, chunk=1024, experts=16, identity=1, top=4, vocab=32768, compute_f32=False):
    """A Lurepel-design stack at sizes that resemble a served model's layers (random-init benchmarks): heads of 128 channels,
    four query heads per key/value head, half of each head rotated, attention inside blocks of `chunk` positions; layers
    alternate a dense gated feed-forward of size ff with a mixture of `experts` experts of size ff / top (+ identity outputs)
    of which every token uses `top`, so both kinds spend the same products per token."""
    from . import engine as E
    heads = max(1, width // 128)
    ff = ff or (width * 4)
    flags = E.ATTN_QK_UNIT_NORM | E.ATTN_V_IS_K | E.ATTN_UNIT_SINK | E.ATTN_HEAD_GATE
    out = []
    for i in range(layers):
        l = E.LayerDesc(mixer=E.MIXER_GQA, heads=heads, kv_heads=max(1, heads // 4), dim=128, vdim=128, scale=128 ** -0.5,
                        attn_flags=flags, mask=E.MASK_CHUNK, window=chunk, rope_dims=64, rope_pairing=1, rope_base=500000.0,
                        rope_factor=8.0, rope_low=1.0, rope_high=4.0, rope_original=8192)
        if i % 2 == 0:
            l.ff_kind, l.ff = E.FF_GELU_TANH, ff
        else:
            l.ff_kind, l.ff, l.experts, l.identity_experts, l.top_k = E.FF_MOE, max(64, ff // top), experts, identity, top
        out.append(l)
    return E.StackDesc(width=width, vocab=vocab, layers=out, compute_f32=int(compute_f32), norm_eps=1e-5, resid_alpha=1.0,
                       logit_softcap=0.0, norm_place=E.NORM_OF_OUTPUT, embed_norm=1, plain_gains=1)


def latanex_stack(width, layers, ff=None, window=1024, experts=16, top=4, groups=(4, 2), vocab=32768, compute_f32=False):
    """A Latanex-design stack at sizes that resemble a served model's layers (random-init benchmarks): heads of 128 channels,
    four query heads per key/value head, a sliding window, capped scores, learned sinks and blended values; every fourth
    layer (the third of each four) is a gated-delta-rule layer with 128 x 128 states and four-tap convolutions; the first
    layer has a dense gated feed-forward of size ff, the others a mixture of `experts` clamped experts of size 3 ff / 16 of
    which every token uses `top` out of the best groups, plus a shared expert of size ff / 4: the products of a dense unit of
    size ff per token."""
    from . import engine as E
    heads = max(1, width // 128)
    ff = ff or (width * 4)
    flags = E.ATTN_QKV_BIAS | E.ATTN_QK_PROJ_NORM | E.ATTN_LEARNED_SINK | E.ATTN_V_BLEND
    out = []
    for i in range(layers):
        if i % 4 == 2:
            l = E.LayerDesc(mixer=E.MIXER_DELTA, heads=heads, kv_heads=max(1, heads // 2), dim=128, vdim=128, conv_taps=4)
        else:
            l = E.LayerDesc(mixer=E.MIXER_GQA, heads=heads, kv_heads=max(1, heads // 4), dim=128, vdim=128, scale=128 ** -0.5,
                            attn_flags=flags, mask=E.MASK_WINDOW, window=window, score_cap=30.0)
        if i == 0:
            l.ff_kind, l.ff = E.FF_SILU, ff
        else:
            l.ff_kind, l.ff, l.ff_limit, l.experts, l.top_k = E.FF_MOE, max(64, 3 * ff // 16), 7.0, experts, top
            l.router_kind, l.expert_kind, l.route_renorm, l.route_scale = E.ROUTER_SIGMOID, E.EXPERT_CLAMPED, 1, 2.5
            l.route_groups, l.route_keep = groups
            l.shared_ff, l.shared_limit = max(64, ff // 4), 7.0
        out.append(l)
    return E.StackDesc(width=width, vocab=vocab, layers=out, compute_f32=int(compute_f32), norm_eps=1e-5, resid_alpha=1.0,
                       norm_place=E.NORM_BOTH_SIDES, norm_kind=E.NORM_TANH, plain_gains=1, embed_scale=1.0, logit_scale=0.25)


def funudra_stack(width, layers, ff=None, vocab=32768, share=False, compute_f32=False):
    """A Funudra-design stack at sizes that resemble a served model's layers (random-init benchmarks).  Two of three layers
    are state-space layers (inner size 2 width in heads of 64 channels, 128 states per channel, eight groups, four-tap
    convolution, eight norm parts); the middle one of each three has two mixers side by side: grouped-query attention (heads
    of 128, four query heads per key/value head, four-tap convolutions on q / k / v, half of each head rotated with linearly
    scaled frequencies, capped scores, entry-wise output gate) and a matrix memory (heads of 64 x 128).  Every layer has a
    relu-squared feed-forward of size ff on the same stream; the embedding table is the output matrix.  share: the second
    half of the layers uses the tensors of the first half."""
    from . import engine as E
    heads = max(1, width // 128)
    ff = ff or (width * 4)
    out = []
    for i in range(layers):
        if i % 3 == 1:
            l = E.LayerDesc(mixer=E.MIXER_GQA, heads=heads, kv_heads=max(1, heads // 4), dim=128, vdim=128, scale=128 ** -0.5,
                            attn_flags=E.ATTN_QKV_BIAS | E.ATTN_QKV_CONV | E.ATTN_OUT_GATE | E.ATTN_OUT_BIAS, conv_taps=4,
                            mask=E.MASK_CAUSAL, window=0, score_cap=30.0, rope_dims=64, rope_pairing=0, rope_base=500000.0,
                            rope_linear=4.0, side_mixer=E.MIXER_MLSTM, side_heads=heads, side_dim=64, side_vdim=128,
                            side_gate_cap=15.0, mix_scale=0.7, side_scale=0.7)
        else:
            mh = max(8, 2 * width // 64)
            l = E.LayerDesc(mixer=E.MIXER_MAMBA2, heads=mh, vdim=64, dim=128, kv_heads=8, norm_groups=8, conv_taps=4)
        l.ff_kind, l.ff = E.FF_RELU2, ff
        if share and i >= (layers + 1) // 2 and (i - (layers + 1) // 2) % 3 == i % 3:
            l.weights_of = i - (layers + 1) // 2 + 1
        out.append(l)
    return E.StackDesc(width=width, vocab=vocab, layers=out, compute_f32=int(compute_f32), norm_eps=1e-5, resid_alpha=1.0,
                       norm_place=E.NORM_PARALLEL, embed_norm=1, plain_gains=1, tie_head=1)


def llama_like(width, layers, ff, vocab=32768):
    """The closest existing decoder at equal width / depth / feed-forward size (comparison arm of the layer-list benchmarks)."""
    heads = max(1, width // 128)
    return ModelDesc(arch=LLAMA, hidden=width, layers=layers, heads=heads, kv_heads=max(1, heads // 4), head_dim=128, ffn=ff,
                     vocab=vocab, max_pos=8192, tie_embeddings=0, norm_eps=1e-5, rope_theta=500000.0)
