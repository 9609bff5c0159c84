"""Parameter inventories (checkpoint names and shapes, in ``parameter_ids`` order) of the model families whose
optimizer step the library runs. Only the inventory matters to the step: names decide the weight-decay group
(src/weight_decay/rule.rs:103-118), shapes give ranks and element counts, order gives the flat layout.

Order and names follow LitGPT::named_parameters (src/model.rs:3905-3953, 4746-4913): embed_tokens, per layer
input_layernorm, q/k/v/o (+ q_norm/k_norm), post_attention_layernorm, the FFN, then norm and an untied lm_head;
on-disk names carry the ``model.`` prefix except lm_head (src/checkpoint_names.rs:14-28).
"""
from __future__ import annotations

from .dpstep import TensorInfo


def _ckpt(name: str) -> str:
    return name if name.startswith("lm_head.") else "model." + name


def _attention(prefix: str, hidden: int, heads: int, kv_heads: int, head_dim: int, qk_norm: bool) -> list[TensorInfo]:
    out = [TensorInfo(f"{prefix}.input_layernorm.weight", (hidden,))]
    for name, rows in (("q_proj", heads * head_dim), ("k_proj", kv_heads * head_dim), ("v_proj", kv_heads * head_dim)):
        out.append(TensorInfo(f"{prefix}.self_attn.{name}.weight", (rows, hidden)))
    out.append(TensorInfo(f"{prefix}.self_attn.o_proj.weight", (hidden, heads * head_dim)))
    if qk_norm:
        out.append(TensorInfo(f"{prefix}.self_attn.q_norm.weight", (head_dim,)))
        out.append(TensorInfo(f"{prefix}.self_attn.k_norm.weight", (head_dim,)))
    out.append(TensorInfo(f"{prefix}.post_attention_layernorm.weight", (hidden,)))
    return out


def _mlp(prefix: str, hidden: int, inter: int) -> list[TensorInfo]:
    return [TensorInfo(f"{prefix}.gate_proj.weight", (inter, hidden)),
            TensorInfo(f"{prefix}.up_proj.weight", (inter, hidden)),
            TensorInfo(f"{prefix}.down_proj.weight", (hidden, inter))]


def _moe(prefix: str, hidden: int, inter: int, experts: int, shared: bool) -> list[TensorInfo]:
    out = [TensorInfo(f"{prefix}.moe.router.gate.weight", (experts, hidden))]
    for e in range(experts):
        out += _mlp(f"{prefix}.moe.experts.{e}", hidden, inter)
    if shared:
        out += _mlp(f"{prefix}.moe.shared_expert", hidden, inter)
    return out


def _finish(body: list[TensorInfo], hidden: int, vocab: int, tied: bool) -> list[TensorInfo]:
    out = [TensorInfo("embed_tokens.weight", (vocab, hidden))] + body + [TensorInfo("norm.weight", (hidden,))]
    if not tied:
        out.append(TensorInfo("lm_head.weight", (vocab, hidden)))
    return [TensorInfo(_ckpt(t.name), t.shape) for t in out]


def dense_gqa(hidden: int, layers: int, heads: int, kv_heads: int, head_dim: int, inter: int, vocab: int,
              tied: bool, qk_norm: bool = False) -> list[TensorInfo]:
    body: list[TensorInfo] = []
    for i in range(layers):
        body += _attention(f"layers.{i}", hidden, heads, kv_heads, head_dim, qk_norm)
        body += _mlp(f"layers.{i}.mlp", hidden, inter)
    return _finish(body, hidden, vocab, tied)


def moe_gqa(hidden: int, layers: int, heads: int, kv_heads: int, head_dim: int, inter: int, experts: int,
            shared: bool, vocab: int, tied: bool = False) -> list[TensorInfo]:
    body: list[TensorInfo] = []
    for i in range(layers):
        body += _attention(f"layers.{i}", hidden, heads, kv_heads, head_dim, False)
        body += _moe(f"layers.{i}", hidden, inter, experts, shared)
    return _finish(body, hidden, vocab, tied)


def hybrid(hidden: int = 384, layers: int = 12, mamba_layers=(0, 2, 4, 6), gdn_layers=(8, 10), expand: int = 2,
           mamba_heads: int = 48, mamba_head_dim: int = 16, d_state: int = 64, d_conv: int = 4, heads: int = 6,
           kv_heads: int = 2, inter: int = 1024, gdn_state: int = 64, gdn_key_heads: int = 2, gdn_value_heads: int = 4,
           vocab: int = 32000, tied: bool = False) -> list[TensorInfo]:
    """Hybrid Mamba3 / GDN / attention inventory.

    Mamba3 names follow src/model.rs:4166-4265 and the block prefix of src/model.rs:4773-4781; GDN names and shapes
    follow src/model/gdn/names.rs:5-18. The Mamba3 tensor SHAPES are fixed inside the un-vendored boostr
    (Mamba3::init); the table below is this library's documented stand-in: d_inner = expand*hidden =
    heads*head_dim, per-head vectors of `heads`, a depthwise conv of width d_conv over d_inner + 2*d_state channels.
    """
    d_inner = expand * hidden
    assert d_inner == mamba_heads * mamba_head_dim
    conv_ch = d_inner + 2 * d_state
    head_dim = hidden // heads
    body: list[TensorInfo] = []
    for i in range(layers):
        p = f"layers.{i}"
        if i in mamba_layers:
            m = f"{p}.mamba3"
            body += [TensorInfo(f"{p}.norm.weight", (hidden,)), TensorInfo(f"{p}.norm.bias", (hidden,)),
                     TensorInfo(f"{m}.in_proj.weight", (2 * d_inner + 2 * d_state + mamba_heads, hidden)),
                     TensorInfo(f"{m}.out_proj.weight", (hidden, d_inner)),
                     TensorInfo(f"{m}.lambda_proj.weight", (mamba_heads, hidden)),
                     TensorInfo(f"{m}.b_bias", (mamba_heads, d_state)), TensorInfo(f"{m}.c_bias", (mamba_heads, d_state)),
                     TensorInfo(f"{m}.dt_bias", (mamba_heads,)), TensorInfo(f"{m}.A_log", (mamba_heads,)),
                     TensorInfo(f"{m}.D", (mamba_heads,)), TensorInfo(f"{m}.bc_norm.weight", (d_state,)),
                     TensorInfo(f"{m}.norm.weight", (d_inner,)),
                     TensorInfo(f"{m}.conv1d.weight", (conv_ch, 1, d_conv)), TensorInfo(f"{m}.conv1d.bias", (conv_ch,))]
        elif i in gdn_layers:
            key_dim, value_dim = gdn_key_heads * gdn_state, gdn_value_heads * gdn_state
            la = f"{p}.linear_attn"
            body += [TensorInfo(f"{p}.input_layernorm.weight", (hidden,)),
                     TensorInfo(f"{la}.in_proj_qkv.weight", (2 * key_dim + value_dim, hidden)),
                     TensorInfo(f"{la}.in_proj_z.weight", (value_dim, hidden)),
                     TensorInfo(f"{la}.alpha_proj.weight", (gdn_value_heads, hidden)),
                     TensorInfo(f"{la}.beta_proj.weight", (gdn_value_heads, hidden)),
                     TensorInfo(f"{la}.out_proj.weight", (hidden, value_dim)),
                     TensorInfo(f"{la}.conv1d.weight", (2 * key_dim + value_dim, 1, d_conv)),
                     TensorInfo(f"{la}.A_log", (gdn_value_heads,)), TensorInfo(f"{la}.dt_bias", (gdn_value_heads,)),
                     TensorInfo(f"{la}.norm.weight", (gdn_state,)),
                     TensorInfo(f"{p}.post_attention_layernorm.weight", (hidden,))]
            body += _mlp(f"{p}.mlp", hidden, inter)
        else:
            body += _attention(p, hidden, heads, kv_heads, head_dim, False)
            body += _mlp(f"{p}.mlp", hidden, inter)
    return _finish(body, hidden, vocab, tied)


# The five parameter sets the step is measured and checked on.
def nano_dense() -> list[TensorInfo]:
    """Dense GQA, hidden 512, 8 layers, 8 heads, 4 KV heads, SwiGLU 2048, vocab 100315, untied."""
    return dense_gqa(512, 8, 8, 4, 64, 2048, 100315, tied=False)


def llama_3_2_1b() -> list[TensorInfo]:
    """models/llama-3.2-1b.yaml:20-40,81-83."""
    return dense_gqa(2048, 16, 32, 8, 64, 8192, 128256, tied=True)


def qwen3_1_7b() -> list[TensorInfo]:
    """models/qwen3-1.7b.yaml:20-48,80-82 (qk_norm: true)."""
    return dense_gqa(2048, 28, 16, 8, 128, 6144, 151936, tied=True, qk_norm=True)


def moe_1b() -> list[TensorInfo]:
    """hidden 1024, 12 layers, 16 heads, 4 KV heads, 8 routed experts of 2816 + one shared, vocab 32000, untied."""
    return moe_gqa(1024, 12, 16, 4, 64, 2816, 8, True, 32000)


PARAM_SETS = {"nano_dense": nano_dense, "llama-3.2-1b": llama_3_2_1b, "qwen3-1.7b": qwen3_1_7b, "moe-1b": moe_1b,
              "hybrid-384": hybrid}
