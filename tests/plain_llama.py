"""A plain, slow Llama: whole sequences, no cache, one function for each part.

This file is the oracle of the test-suite.  It shares no code with the
``rllm_b200`` package: it reads ``config.json`` with ``json`` and the weights
with the ``safetensors`` library, and computes everything on the CPU in
float64 (``DTYPE``), one sequence at a time, over the whole sequence.

It rests on the formulas of ghyathmoussa/rLLM's model code, cited function by
function below (paths are relative to the reference's root).  The reference's
model needs a Rust toolchain and the Candle crate, neither of which exists on
the machines these tests run on, so the oracle could not be compared with the
reference's own output; it rests on the formulas alone.

Where the reference drops a value that the checkpoints of this architecture
need (``rms_norm_eps`` hard-coded at crates/rllm-model/src/llama.rs:183,
``rope_scaling`` left empty at crates/rllm-model/src/hf_config.rs:68), the
oracle takes the value from ``config.json``; the llama3 frequency rescaling is
the published rule of the Llama 3.1 release, restated in ``rope_inv_freq``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

DTYPE = torch.float64


# ----------------------------------------------------------------------------
# reading a model folder
# ----------------------------------------------------------------------------
def read_model_dir(model_dir: str, round_to: Optional[torch.dtype] = None) -> "PlainLlama":
    """config.json + model.safetensors -> PlainLlama.

    ``round_to=torch.bfloat16`` rounds every matrix to bfloat16 first (what an
    engine running in bfloat16 holds), then computes in float64 all the same.
    """
    from safetensors import safe_open

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            if round_to is not None and t.dtype.is_floating_point and t.dim() >= 2:
                t = t.to(round_to)
            tensors[name] = t.to(DTYPE) if t.dtype.is_floating_point else t
    return PlainLlama(cfg, tensors)


# ----------------------------------------------------------------------------
# the parts, one function each
# ----------------------------------------------------------------------------
def embedding(table: torch.Tensor, token_ids: Sequence[int]) -> torch.Tensor:
    """Row gather, no scaling (crates/rllm-model/src/llama.rs:329-337)."""
    return table[torch.tensor(list(token_ids), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w, eps inside the root, the weight as it is
    (crates/rllm-model/src/layers.rs:133-140)."""
    variance = (x * x).mean(dim=-1, keepdim=True) + eps
    return x / variance.sqrt() * weight


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x . W^T with W stored [out, in], no bias
    (crates/rllm-model/src/layers.rs:162-175)."""
    return x @ weight.t()


def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """f_i = theta^(-2i/d) for i < d/2 (crates/rllm-model/src/rope.rs:13-15).

    With ``rope_scaling`` of type llama3 every f_i is rescaled once by its
    wavelength 2*pi/f_i: shorter than orig/high_freq_factor: kept; longer than
    orig/low_freq_factor: divided by ``factor``; between: blended linearly in
    orig/wavelength.
    """
    idx = torch.arange(0, head_dim, 2, dtype=torch.float64)
    inv = 1.0 / (float(theta) ** (idx / head_dim))
    if not scaling:
        return inv
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return inv
    assert kind == "llama3", kind
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = []
    for f in inv.tolist():
        wavelen = 2.0 * math.pi / f
        if wavelen < orig / high:
            out.append(f)
        elif wavelen > orig / low:
            out.append(f / factor)
        else:
            smooth = (orig / wavelen - low) / (high - low)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return torch.tensor(out, dtype=torch.float64)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate-half convention on [T, heads, d]: out = x*cos + rotate_half(x)*sin
    with rotate_half(x) = [-x2, x1] and the angle table repeated over both
    halves (crates/rllm-model/src/rope.rs:57-82)."""
    angles = positions.to(torch.float64)[:, None] * inv_freq[None, :]      # [T, d/2]
    cos = torch.cat([angles.cos(), angles.cos()], dim=-1)[:, None, :]
    sin = torch.cat([angles.sin(), angles.sin()], dim=-1)[:, None, :]
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    rotated = torch.cat([-x2, x1], dim=-1)
    return x * cos + rotated * sin


def attention_scores_mask(num_q: int, q_positions: torch.Tensor, num_k: int,
                          window: Optional[int]) -> torch.Tensor:
    """True where a query may see a key: key position <= query position
    (causal, crates/rllm-model/src/layers.rs:625-633) and, with a window w,
    key position > query position - w."""
    kpos = torch.arange(num_k)[None, :]
    qpos = q_positions[:, None]
    ok = kpos <= qpos
    if window is not None:
        ok = ok & (kpos > qpos - window)
    return ok


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_positions: torch.Tensor,
              window: Optional[int] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Grouped-query softmax attention over a whole sequence.

    q [Tq, nq, d], k and v [Tk, nkv, d]; key j has position j.  kv head of query
    head h is h*nkv/nq (crates/rllm-kernels/src/cuda/paged_attention.cu:113,
    the same map as repeat_kv, crates/rllm-model/src/layers.rs:609-622);
    scores are scaled by 1/sqrt(d) (crates/rllm-model/src/layers.rs:326-329),
    softmax is over the keys (:339), then P.V and heads are concatenated
    (:340-344).
    """
    tq, nq, d = q.shape
    tk, nkv, _ = k.shape
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    mask = attention_scores_mask(tq, q_positions, tk, window)
    out = torch.empty(tq, nq, v.shape[-1], dtype=q.dtype)
    for h in range(nq):
        kvh = h * nkv // nq
        s = (q[:, h, :] @ k[:, kvh, :].t()) * scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kvh, :]
    return out.reshape(tq, nq * v.shape[-1])


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def gated_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
              w_down: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) (crates/rllm-model/src/layers.rs:214-220)."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


# ----------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------
class PlainLlama:
    def __init__(self, cfg: dict, tensors: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.t = tensors
        self.layers = int(cfg["num_hidden_layers"])
        self.nq = int(cfg["num_attention_heads"])
        self.nkv = int(cfg.get("num_key_value_heads", self.nq))
        self.hidden = int(cfg["hidden_size"])
        self.d = int(cfg.get("head_dim", self.hidden // self.nq))
        self.eps = float(cfg.get("rms_norm_eps", 1e-6))
        self.vocab = int(cfg["vocab_size"])
        self.inv_freq = rope_inv_freq(self.d, float(cfg.get("rope_theta", 10000.0)),
                                      cfg.get("rope_scaling"))

    def attention_part(self, i: int, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """q/k/v projections, head split, RoPE on q and k, attention, o_proj
        (crates/rllm-model/src/layers.rs:280-347)."""
        p = f"model.layers.{i}.self_attn."
        t = x.shape[0]
        q = linear(x, self.t[p + "q_proj.weight"]).reshape(t, self.nq, self.d)
        k = linear(x, self.t[p + "k_proj.weight"]).reshape(t, self.nkv, self.d)
        v = linear(x, self.t[p + "v_proj.weight"]).reshape(t, self.nkv, self.d)
        q = apply_rope(q, positions, self.inv_freq)
        k = apply_rope(k, positions, self.inv_freq)
        a = attention(q, k, v, positions)
        return linear(a, self.t[p + "o_proj.weight"])

    def mlp_part(self, i: int, x: torch.Tensor) -> torch.Tensor:
        p = f"model.layers.{i}.mlp."
        return gated_mlp(x, self.t[p + "gate_proj.weight"], self.t[p + "up_proj.weight"],
                         self.t[p + "down_proj.weight"])

    def decoder_layer(self, i: int, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """h = x + attn(norm_in(x)); out = h + mlp(norm_post(h))
        (crates/rllm-model/src/layers.rs:677-699)."""
        p = f"model.layers.{i}."
        h = x + self.attention_part(i, rms_norm(x, self.t[p + "input_layernorm.weight"], self.eps),
                                    positions)
        return h + self.mlp_part(i, rms_norm(h, self.t[p + "post_attention_layernorm.weight"],
                                             self.eps))

    def head_weight(self) -> torch.Tensor:
        """lm_head.weight if the file has it, else the embedding table
        (crates/rllm-model/src/llama.rs:174-180)."""
        return self.t.get("lm_head.weight", self.t["model.embed_tokens.weight"])

    def logits(self, token_ids: Sequence[int]) -> torch.Tensor:
        """Logits [T, vocab] at every position of one whole sequence
        (crates/rllm-model/src/llama.rs:283-326 and :57-70)."""
        x = embedding(self.t["model.embed_tokens.weight"], token_ids)
        positions = torch.arange(len(token_ids))
        for i in range(self.layers):
            x = self.decoder_layer(i, x, positions)
        x = rms_norm(x, self.t["model.norm.weight"], self.eps)
        return linear(x, self.head_weight())

    def logits_at(self, token_ids: Sequence[int], rows: Sequence[int]) -> torch.Tensor:
        """The rows ``rows`` of ``logits(token_ids)``: the output product on those rows only (a large
        vocabulary makes it the most expensive part of the whole-sequence oracle)."""
        x = embedding(self.t["model.embed_tokens.weight"], token_ids)
        positions = torch.arange(len(token_ids))
        for i in range(self.layers):
            x = self.decoder_layer(i, x, positions)
        x = rms_norm(x[list(rows)], self.t["model.norm.weight"], self.eps)
        return linear(x, self.head_weight())

    def greedy(self, prompt: Sequence[int], max_tokens: int) -> List[int]:
        """Greedy continuation by recomputing the whole sequence each step; the
        lowest index wins a tie."""
        tokens = list(prompt)
        out = []
        for _ in range(max_tokens):
            row = self.logits(tokens)[-1]
            nxt = int(torch.argmax(row))           # torch.argmax returns the first maximum
            out.append(nxt)
            tokens.append(nxt)
        return out


# ----------------------------------------------------------------------------
# plain sampling (numpy, one row at a time)
# ----------------------------------------------------------------------------
def philox4x32_10(counter: Sequence[int], key: Sequence[int]) -> List[int]:
    """The Philox-4x32 block function with 10 rounds (Salmon et al., SC'11)."""
    m0, m1 = 0xD2511F53, 0xCD9E8D57
    w0, w1 = 0x9E3779B9, 0xBB67AE85
    c = [int(x) & 0xFFFFFFFF for x in counter]
    k = [int(x) & 0xFFFFFFFF for x in key]
    for _ in range(10):
        p0 = m0 * c[0]
        p1 = m1 * c[2]
        hi0, lo0 = p0 >> 32, p0 & 0xFFFFFFFF
        hi1, lo1 = p1 >> 32, p1 & 0xFFFFFFFF
        c = [(hi1 ^ c[1] ^ k[0]) & 0xFFFFFFFF, lo1, (hi0 ^ c[3] ^ k[1]) & 0xFFFFFFFF, lo0]
        k = [(k[0] + w0) & 0xFFFFFFFF, (k[1] + w1) & 0xFFFFFFFF]
    return c


def uniform_for(seed: int, index: int) -> float:
    """The uniform number in [0, 1) that decides generated token ``index`` of a
    request with this seed: top 24 bits of the first Philox word."""
    word = philox4x32_10([index & 0xFFFFFFFF, (index >> 32) & 0xFFFFFFFF, 0, 0],
                         [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF])[0]
    return (word >> 8) * (1.0 / 16777216.0)


def process_logits(logits: np.ndarray, *, context: Sequence[int] = (), logit_bias=None,
                   repetition_penalty: float = 1.0, frequency_penalty: float = 0.0,
                   presence_penalty: float = 0.0, allowed_token_ids=None,
                   suppress: Sequence[int] = (), temperature: float = 1.0, top_k: int = -1,
                   top_p: float = 1.0, min_p: float = 0.0) -> np.ndarray:
    """The reference's order of logits processors
    (crates/rllm-sampling/src/sampler.rs:62-133 with the functions of
    crates/rllm-sampling/src/logits.rs:5-185), in float32 like the reference.
    Two deliberate differences, shared with the engine: top_k keeps the k
    largest values and their ties (the reference's threshold at logits.rs:26-31
    is the (k+1)-th largest, which keeps k+1), and top_p keeps every tie of the
    last value it takes (the reference cuts among equal values in sort order)."""
    x = np.array(logits, dtype=np.float32).copy()
    n = x.shape[0]
    if logit_bias:
        for tid, b in logit_bias.items():
            if 0 <= tid < n:
                x[tid] += np.float32(b)
    ctx = [t for t in context if 0 <= t < n]
    if ctx:
        if repetition_penalty != 1.0:
            # applied once per occurrence, like the reference's loop (logits.rs:95-110)
            for t in ctx:
                x[t] = x[t] / np.float32(repetition_penalty) if x[t] > 0 else x[t] * np.float32(repetition_penalty)
        if frequency_penalty != 0.0:
            counts: Dict[int, int] = {}
            for t in ctx:
                counts[t] = counts.get(t, 0) + 1
            for t, c in counts.items():
                x[t] -= np.float32(frequency_penalty) * np.float32(c)
        if presence_penalty != 0.0:
            for t in set(ctx):
                x[t] -= np.float32(presence_penalty)
    if allowed_token_ids:
        keep = np.zeros(n, dtype=bool)
        keep[[t for t in allowed_token_ids if 0 <= t < n]] = True
        x[~keep] = -np.inf
    for t in suppress:
        if 0 <= t < n:
            x[t] = -np.inf
    greedy = temperature <= 0.0 or top_k == 1
    if greedy:
        return x
    if abs(temperature - 1.0) >= np.finfo(np.float32).eps:
        x = x * np.float32(1.0 / np.float32(temperature))
    if 0 < top_k < n:
        kth = np.sort(x)[::-1][top_k - 1]        # keep the k largest (and their ties)
        x[x < kth] = -np.inf
    if 0.0 < top_p < 1.0:
        order = np.argsort(-x, kind="stable")
        order = order[x[order] > -np.inf]
        vals = x[order].astype(np.float64)
        probs = np.exp(vals - vals[0])
        probs /= probs.sum()
        cum = np.cumsum(probs)
        cutoff = int(np.searchsorted(cum, top_p, side="left")) + 1     # first prefix with cum >= p
        cutoff = min(cutoff, len(order))
        last = vals[cutoff - 1]
        x[x < np.float32(last)] = -np.inf                               # ties of the last value stay
    if min_p > 0.0:
        m = x.max()
        if m > -np.inf:
            x[x < np.float32(math.log(min_p)) + m] = -np.inf
    return x


def sample_row(processed: np.ndarray, temperature: float, top_k: int, u: float) -> int:
    """Greedy when temperature <= 0 or top_k == 1 (sampler.rs:117), else
    softmax and the first index whose running sum exceeds u (sampler.rs:194-214
    has ``>=``, which would draw a masked token 0 when u is 0).  Greedy ties go
    to the lowest index."""
    if temperature <= 0.0 or top_k == 1:
        return int(np.argmax(processed))
    x = processed.astype(np.float64)
    e = np.exp(x - x.max())
    p = e / e.sum()
    cum = np.cumsum(p)
    idx = int(np.searchsorted(cum, u, side="right"))
    return min(idx, len(p) - 1)


def logprob_of(logits: np.ndarray, token: int) -> float:
    """Natural-log probability of ``token`` under softmax(logits):
    logit - (max + ln sum exp(logit - max)) (crates/rllm-sampling/src/logprobs.rs:5-28), in float64."""
    x = np.asarray(logits, dtype=np.float64)
    m = x.max()
    if m == -np.inf or not 0 <= token < len(x):
        return -np.inf
    return float(x[token] - (m + math.log(np.exp(x - m).sum())))


def top_logprobs(logits: np.ndarray, n: int) -> List[tuple]:
    """The n likeliest tokens as (id, log-probability), descending (crates/rllm-sampling/src/logprobs.rs:34-70);
    -inf logits are left out; among equals the lower index comes first (the reference sorts unstably)."""
    x = np.asarray(logits, dtype=np.float64)
    m = x.max()
    if n <= 0 or m == -np.inf:
        return []
    log_z = m + math.log(np.exp(x - m).sum())
    order = sorted((i for i in range(len(x)) if x[i] != -np.inf), key=lambda i: (-x[i], i))[:n]
    return [(int(i), float(x[i] - log_z)) for i in order]
