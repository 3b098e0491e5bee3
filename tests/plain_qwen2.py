"""A plain, slow, whole-sequence implementation of the Qwen2 dense decoder.

Written from the formulas of the reference's model code; each function cites the
lines it restates.  No cache, no batching tricks, one function per part, float32
(or float64) torch on the CPU.  It shares no code with the package: the tests
compare the engine against it.  `tests/golden/` holds the outputs of one
comparison of this file with the reference's own pure-torch model
(pico_vllm/legacy/model.py) on a tiny random model, and the script that made them.

Weights are passed as a dict keyed by the tensor names of the model folder
(`model.layers.{i}.self_attn.q_proj.weight`, …; pico_vllm/weights.py:18-68).
"""
import math

import torch


def embed(ids, table):
    """x = E[ids]  (pico_vllm/model.py:405,427)."""
    return table[ids]


def rms_norm(x, weight, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w  (pico_vllm/model.py:57-66, pico_vllm/RMSNorm.py:22-34)."""
    var = x.pow(2).mean(-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def rotary_angles(positions, head_dim, theta, dtype=torch.float32):
    """inv_freq_i = 1/theta^(2i/hd); angle = position * inv_freq  (pico_vllm/model.py:80-86)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).to(dtype) / head_dim))
    ang = torch.outer(positions.to(dtype), inv_freq)
    return ang.cos(), ang.sin()  # [T, hd/2] each


def apply_rotary(x, cos, sin):
    """Half-split rotation: x1' = x1 c - x2 s, x2' = x2 c + x1 s  (pico_vllm/model.py:116-124).

    x: [T, heads, hd]; cos, sin: [T, hd/2].
    """
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def attention_scores_softmax_pv(q, k, v, positions, window=None):
    """Causal attention of one sequence with grouped heads.

    Query head j reads key/value head j // g (pico_vllm/kernels/attention.py:31,139);
    s = q.k / sqrt(hd) (pico_vllm/kernels/attention.py:92,231); key n is visible to the
    query at position p iff n <= p (pico_vllm/kernels/attention.py:193-198), and, when a
    window W is given, also n > p - W (the last W keys, the query's own included; the
    reference has no window, the rule is the config key's meaning); softmax over
    the visible keys; o = P.V (pico_vllm/kernels/attention.py:189-213).
    q: [T, nh, hd], k, v: [T, nkv, hd] for positions 0..T-1 in order.
    """
    T, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.empty_like(q)
    key_pos = positions[None, :]
    qry_pos = positions[:, None]
    visible = key_pos <= qry_pos
    if window is not None:
        visible = visible & (key_pos > qry_pos - window)
    for j in range(nh):
        kj, vj = k[:, j // g, :], v[:, j // g, :]
        s = (q[:, j, :] @ kj.T) / math.sqrt(hd)
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, j, :] = p @ vj
    return out


def attention_block(h, w, prefix, positions, cfg, window):
    """qkv projection with bias, rotation of q and k, attention, output projection without
    bias (pico_vllm/model.py:147-152, 200-225; separate q/k/v matrices as in
    pico_vllm/legacy/model.py:80-84)."""
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = h.shape[0]
    q = (h @ w[prefix + "q_proj.weight"].T + w[prefix + "q_proj.bias"]).view(T, nh, hd)
    k = (h @ w[prefix + "k_proj.weight"].T + w[prefix + "k_proj.bias"]).view(T, nkv, hd)
    v = (h @ w[prefix + "v_proj.weight"].T + w[prefix + "v_proj.bias"]).view(T, nkv, hd)
    cos, sin = rotary_angles(positions, hd, cfg["rope_theta"], dtype=h.dtype)
    q, k = apply_rotary(q, cos, sin), apply_rotary(k, cos, sin)
    o = attention_scores_softmax_pv(q, k, v, positions, window)
    return o.reshape(T, nh * hd) @ w[prefix + "o_proj.weight"].T


def swiglu_mlp(h, w, prefix):
    """down( silu(gate(h)) * up(h) ), silu(g) = g * sigmoid(g)
    (pico_vllm/model.py:314-318; pico_vllm/kernels/swiglu.py:36-41)."""
    g = h @ w[prefix + "gate_proj.weight"].T
    u = h @ w[prefix + "up_proj.weight"].T
    return (g * torch.sigmoid(g) * u) @ w[prefix + "down_proj.weight"].T


def decoder_layer(x, w, i, positions, cfg):
    """x += attn(norm1(x)); x += mlp(norm2(x))  (pico_vllm/model.py:361-374)."""
    p = f"model.layers.{i}."
    eps = cfg["rms_norm_eps"]
    window = cfg.get("layer_windows", [None] * cfg["num_hidden_layers"])[i]
    x = x + attention_block(rms_norm(x, w[p + "input_layernorm.weight"], eps), w,
                            p + "self_attn.", positions, cfg, window)
    x = x + swiglu_mlp(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    return x


def lm_head(h, w, cfg):
    """logits = h.E^T when tied; the separate lm_head matrix otherwise
    (pico_vllm/model.py:445 for the tied case; pico_vllm/legacy/model.py:223-226 for both)."""
    if cfg["tie_word_embeddings"]:
        return h @ w["model.embed_tokens.weight"].T
    return h @ w["lm_head.weight"].T


def last_hidden_states(ids, w, cfg, dtype=torch.float32):
    """The normed states [T, width] that the head multiplies, for one whole sequence of token ids:
    embedding, every layer, last norm (pico_vllm/model.py:427-444).  For vocabularies so large
    that logits of every position would not fit, callers apply :func:`lm_head` to the rows they want."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    w = {k: v.to(dtype) for k, v in w.items()}
    positions = torch.arange(ids.shape[0])
    x = embed(ids, w["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, positions, cfg)
    return rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])


def forward(ids, w, cfg, dtype=torch.float32):
    """Logits [T, vocab] of one whole sequence of token ids (list or 1-D tensor)
    (pico_vllm/model.py:427-445)."""
    w = {k: v.to(dtype) for k, v in w.items()}
    return lm_head(last_hidden_states(ids, w, cfg, dtype), w, cfg)


def greedy_generate(prompt, w, cfg, n_new, dtype=torch.float32):
    """Greedy continuation by recomputing the whole sequence for every token
    (argmax: pico_vllm/sampler.py:3-8)."""
    ids = list(prompt)
    for _ in range(n_new):
        logits = forward(ids, w, cfg, dtype)
        ids.append(int(torch.argmax(logits[-1])))
    return ids[len(prompt):]


def softmax_temperature(logits, temperature):
    """probs = softmax(logits / T)  (pico_vllm/sampler.py:16)."""
    return torch.softmax(logits / temperature, dim=-1)


def top_p_filter(probs, top_p):
    """Sort descending, cumulative sum, drop where cum - p >= top_p, renormalise
    (pico_vllm/sampler.py:26-33).  Returns probabilities in vocabulary order."""
    sp, si = torch.sort(probs, descending=True, dim=-1)
    cum = torch.cumsum(sp, dim=-1)
    sp = sp.masked_fill(cum - sp >= top_p, 0.0)
    sp = sp / sp.sum(dim=-1, keepdim=True)
    out = torch.zeros_like(probs)
    out.scatter_(-1, si, sp)
    return out


def config_dict(vocab_size, hidden_size, num_hidden_layers, num_attention_heads, num_key_value_heads,
                intermediate_size, rms_norm_eps, rope_theta, tie_word_embeddings, head_dim=None,
                layer_windows=None):
    """The sizes the functions above read, as a plain dict."""
    return dict(vocab_size=vocab_size, hidden_size=hidden_size, num_hidden_layers=num_hidden_layers,
                num_attention_heads=num_attention_heads, num_key_value_heads=num_key_value_heads,
                head_dim=head_dim or hidden_size // num_attention_heads,
                intermediate_size=intermediate_size, rms_norm_eps=rms_norm_eps, rope_theta=rope_theta,
                tie_word_embeddings=tie_word_embeddings,
                layer_windows=layer_windows or [None] * num_hidden_layers)


def random_weights(cfg, seed, std=0.02):
    """Seeded weights by tensor name: matrices and biases ~N(0, std), norm weights 1+N(0, std)."""
    g = torch.Generator().manual_seed(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def n(*shape):
        return torch.randn(*shape, generator=g) * std

    w = {"model.embed_tokens.weight": n(V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "self_attn.q_proj.weight"] = n(nh * hd, H)
        w[p + "self_attn.q_proj.bias"] = n(nh * hd)
        w[p + "self_attn.k_proj.weight"] = n(nkv * hd, H)
        w[p + "self_attn.k_proj.bias"] = n(nkv * hd)
        w[p + "self_attn.v_proj.weight"] = n(nkv * hd, H)
        w[p + "self_attn.v_proj.bias"] = n(nkv * hd)
        w[p + "self_attn.o_proj.weight"] = n(H, nh * hd)
        w[p + "mlp.gate_proj.weight"] = n(I, H)
        w[p + "mlp.up_proj.weight"] = n(I, H)
        w[p + "mlp.down_proj.weight"] = n(H, I)
        w[p + "input_layernorm.weight"] = 1.0 + n(H)
        w[p + "post_attention_layernorm.weight"] = 1.0 + n(H)
    w["model.norm.weight"] = 1.0 + n(H)
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = n(V, H)
    return w
