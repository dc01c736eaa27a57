"""Plain, slow Llama decoder used as the oracle of the test-suite.

It rests on the formulas of integrallis/models alone: that project is a Java 25
library whose numeric core lives in an external artifact, and neither a JVM nor
its build tool is installed next to these tests, so its code cannot be compiled
or imported here.  Every function below restates one formula and cites the file
and lines (paths inside integrallis/models) it was taken from.

Whole sequences only, no cache, one function per part, CPU tensors.  Nothing in
this file imports the engine, and the engine imports nothing from here.

Two deliberate differences from the Java code, both forced by the model-folder
format (config.json + safetensors) instead of GGUF:
  * rotary pairs are split-half, (x[i], x[i + hd/2]) -- safetensors rows are not
    permuted the way GGUF converters permute them, so this is the reference's
    "NeoX" routine applied to unpermuted weights;
  * "llama3" frequency scaling is expressed through the reference's per-pair
    divisor hook (a factor that divides a pair's angle), which the Java Llama
    path carries but never fills in.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# --------------------------------------------------------------------------- files

_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """Reads every tensor of one safetensors file; bfloat16 and float16 are widened to float32."""
    raw = Path(path).read_bytes()
    (header_len,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + header_len])
    data = raw[8 + header_len :]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        begin, end = info["data_offsets"]
        chunk = data[begin:end]
        shape = tuple(info["shape"])
        if info["dtype"] == "BF16":
            u16 = np.frombuffer(chunk, dtype=np.uint16).astype(np.uint32) << 16
            arr = u16.view(np.float32)
        else:
            arr = np.frombuffer(chunk, dtype=_ST_DTYPES[info["dtype"]])
        t = torch.from_numpy(arr.copy()).reshape(shape)
        out[name] = t.float() if t.is_floating_point() else t
    return out


def read_model_folder(folder):
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = read_safetensors(folder / "model.safetensors")
    return config, weights


# --------------------------------------------------------------------------- parts

def embed(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """x = E[token, :]; the llama embedding scale is 1 (backend-java/.../llama/LlamaForwardPass.java:1024-1025)."""
    return table[tokens]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """sumSq = sum x_i^2; rms = sqrt(sumSq/size + eps); out_i = x_i * (1/rms) * w_i
    (backend-java/.../ops/TensorOps.java:45-58, that multiplication order)."""
    size = x.shape[-1]
    sum_sq = (x * x).sum(dim=-1, keepdim=True)
    rms = torch.sqrt(sum_sq / size + eps)
    scale = 1.0 / rms
    return x * scale * weight


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """out[r] = sum_c W[r, c] * x[c] for a row-major [rows, cols] matrix
    (backend-java/.../ops/TensorOps.java:61-63); the optional bias is added afterwards
    (backend-java/.../llama/LlamaForwardPass.java:1065-1067)."""
    out = x @ weight.t()
    if bias is not None:
        out = out + bias
    return out


def rope_pair_frequencies(rotary_dim: int, theta: float) -> torch.Tensor:
    """freq_i = (float)(1 / theta^(2i / rotary_dim)), the power taken in double
    (backend-java/.../ops/RotaryTable.java:70-72)."""
    pairs = rotary_dim // 2
    freqs = [1.0 / math.pow(float(theta), (2.0 * i) / rotary_dim) for i in range(pairs)]
    return torch.tensor(freqs, dtype=torch.float64).float()


def llama3_pair_divisors(freqs: torch.Tensor, factor: float, low_freq_factor: float,
                         high_freq_factor: float, original_max_position: int) -> torch.Tensor:
    """Per-pair divisors of the angle (the hook of backend-java/.../ops/RotaryTable.java:48-66,177-186).

    wavelength = 2*pi / freq.  Shorter than original/high: untouched (divisor 1).  Longer than
    original/low: divided by `factor`.  Between: freq' = (1-s)*freq/factor + s*freq with
    s = (original/wavelength - low) / (high - low); the divisor is freq / freq'.
    """
    out = []
    for f in freqs.double().tolist():
        wavelength = 2.0 * math.pi / f
        if wavelength < original_max_position / high_freq_factor:
            out.append(1.0)
        elif wavelength > original_max_position / low_freq_factor:
            out.append(float(factor))
        else:
            s = (original_max_position / wavelength - low_freq_factor) / (high_freq_factor - low_freq_factor)
            scaled = (1.0 - s) * f / factor + s * f
            out.append(f / scaled)
    return torch.tensor(out, dtype=torch.float64).float()


def rope_cos_sin(positions: torch.Tensor, freqs: torch.Tensor, divisors: torch.Tensor | None,
                 frequency_scale: float = 1.0):
    """angle = (pos * frequencyScale) * freq_i / divisor_i in float; cos and sin taken in double and
    rounded to float (backend-java/.../ops/RotaryTable.java:177-186)."""
    scaled_position = positions.float() * torch.tensor(frequency_scale, dtype=torch.float32)
    angle = scaled_position[:, None] * freqs[None, :]
    if divisors is not None:
        angle = angle / divisors[None, :]
    angle64 = angle.double()
    return torch.cos(angle64).float(), torch.sin(angle64).float()


def rope_rotate_split_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, head_dim]; pair i is (x[i], x[i + pairs]) over the first 2*pairs coordinates:
    x0' = x0*c - x1*s, x1' = x0*s + x1*c (backend-java/.../ops/TensorOps.java:1384-1404,1481-1486)."""
    pairs = cos.shape[-1]
    x0 = x[..., :pairs]
    x1 = x[..., pairs : 2 * pairs]
    c = cos[:, None, :]
    s = sin[:, None, :]
    rotated = torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)
    return torch.cat([rotated, x[..., 2 * pairs :]], dim=-1)


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """q: [T, nh, hd]; k, v: [T, nkv, hd] -> [T, nh*hd].

    kvHead = head / (nh/nkv); score_p = dot(q_h, K[p, kvHead]) * (float)(1/sqrt(hd)) for the
    visible p (dot first, then scale); causal by construction, p <= pos, and with a window of n
    only the n positions that end at the query (backend-java/.../llama/LlamaConfig.java:184-195);
    softmax with max subtraction, exp, sum, multiply by 1/sum
    (backend-java/.../ops/TensorOps.java:1247-1279); out_h = sum_p prob_p * V[p, kvHead]
    (backend-java/.../llama/LlamaForwardPass.java:1543-1593,1595-1670).
    """
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = torch.tensor(1.0 / math.sqrt(hd), dtype=torch.float64).to(q.dtype)
    out = torch.zeros(T, nh, hd, dtype=q.dtype)
    for head in range(nh):
        kv_head = head // group
        for pos in range(T):
            first = 0 if window is None else max(0, pos - window + 1)
            keys = k[first : pos + 1, kv_head, :]
            scores = (keys @ q[pos, head, :]) * scale
            m = scores.max()
            e = torch.exp(scores - m)
            probs = e * (1.0 / e.sum())
            out[pos, head, :] = probs @ v[first : pos + 1, kv_head, :]
    return out.reshape(T, nh * hd)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(g) * u with silu(z) = z / (1 + exp(-z)) (backend-java/.../ops/TensorOps.java:1407-1425)."""
    return (gate / (1.0 + torch.exp(-gate))) * up


def gelu_glu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """0.5 g (1 + tanh(0.7978845608 g (1 + 0.044715 g^2))) * up (backend-java/.../ops/TensorOps.java:1427-1449;
    the reference reads tanh from a table, this is the function the table samples)."""
    inner = 0.7978845608028654 * gate * (1.0 + 0.044715 * gate * gate)
    return 0.5 * gate * (1.0 + torch.tanh(inner)) * up


def softcap_logits(logits: torch.Tensor, softcap: float) -> torch.Tensor:
    """softcap * tanh(logits / softcap); 0 means none (backend-java/.../llama/LlamaForwardPass.java:1751-1764)."""
    if softcap == 0.0:
        return logits
    return softcap * torch.tanh(logits / softcap)


def feed_forward(xn, w_gate, w_up, w_down, b_gate=None, b_up=None, b_down=None):
    """d = Wd . (silu(Wg.xn) * (Wu.xn)) (backend-java/.../llama/LlamaForwardPass.java:1166-1178)."""
    return linear(swiglu(linear(xn, w_gate, b_gate), linear(xn, w_up, b_up)), w_down, b_down)


# --------------------------------------------------------------------------- model

def rope_tables_from_config(config: dict, positions: torch.Tensor):
    hd = head_dim_of(config)
    params = config.get("rope_parameters") or {}
    theta = config.get("rope_theta", params.get("rope_theta", 10000.0))
    scaling = config.get("rope_scaling")
    if scaling is None and params.get("rope_type", "default") != "default":
        scaling = params
    freqs = rope_pair_frequencies(hd, theta)
    divisors = None
    frequency_scale = 1.0
    if scaling is not None:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind == "llama3":
            divisors = llama3_pair_divisors(
                freqs, scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"],
                scaling["original_max_position_embeddings"])
        elif kind == "linear":
            # frequencyScale = 1/factor (backend-java/.../llama/LlamaConfig.java:302-311)
            frequency_scale = 1.0 / float(scaling["factor"])
        elif kind not in (None, "default"):
            raise ValueError(f"plain implementation has no rope scaling {kind!r}")
    return rope_cos_sin(positions, freqs, divisors, frequency_scale)


def head_dim_of(config: dict) -> int:
    return config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"]


def forward(config: dict, weights: dict[str, torch.Tensor], tokens, dtype=torch.float32,
            return_hidden: bool = False) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence, every position
    (layer order: backend-java/.../llama/LlamaForwardPass.java:1028-1196)."""
    w = {k: (t.to(dtype) if t.is_floating_point() else t) for k, t in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.numel()
    nh = config["num_attention_heads"]
    nkv = config.get("num_key_value_heads") or nh
    hd = head_dim_of(config)
    eps = config["rms_norm_eps"]
    window = config.get("sliding_window")
    cos, sin = rope_tables_from_config(config, torch.arange(T))
    cos, sin = cos.to(dtype), sin.to(dtype)

    x = embed(w["model.embed_tokens.weight"], tokens)
    hidden = []
    for layer in range(config["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        xn = rms_norm(x, w[p + "input_layernorm.weight"], eps)
        q = linear(xn, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias")).reshape(T, nh, hd)
        k = linear(xn, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias")).reshape(T, nkv, hd)
        v = linear(xn, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias")).reshape(T, nkv, hd)
        q = rope_rotate_split_half(q, cos, sin)
        k = rope_rotate_split_half(k, cos, sin)
        attn = causal_gqa_attention(q, k, v, window)
        x = x + linear(attn, w[p + "self_attn.o_proj.weight"], w.get(p + "self_attn.o_proj.bias"))
        xn = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + feed_forward(
            xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"],
            w.get(p + "mlp.gate_proj.bias"), w.get(p + "mlp.up_proj.bias"), w.get(p + "mlp.down_proj.bias"))
        hidden.append(x)
    xn = rms_norm(x, w["model.norm.weight"], eps)
    # tied output: the embedding matrix stands in when there is no output matrix
    # (backend-java/.../llama/LlamaWeights.java:83-89)
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    logits = linear(xn, head)
    if return_hidden:
        return logits, hidden
    return logits


# --------------------------------------------------------------------------- sampling (plain)

def plain_argmax(logits) -> int:
    """First maximum wins (models-runtime/.../Sampler.java:244-252)."""
    best = 0
    values = [float(v) for v in logits]
    for i in range(1, len(values)):
        if values[i] > values[best]:
            best = i
    return best


def plain_candidates(logits, previous_tokens, temperature, top_k, top_p, repetition_penalty):
    """The reference's filtered distribution (models-runtime/.../Sampler.java:78-151,174-205):
    repetition penalty once per earlier occurrence (positive / r, else * r), divide by the
    temperature, softmax over the whole vocabulary, the k most probable with ties to the lower id,
    the shortest prefix of these whose mass reaches top_p (the crossing token included).
    Returns (ids in descending order, their un-renormalised probabilities)."""
    adjusted = np.asarray(logits, dtype=np.float32).copy()
    if repetition_penalty > 1.0:
        r = np.float32(repetition_penalty)
        for t in previous_tokens:
            if 0 <= t < adjusted.size:
                adjusted[t] = adjusted[t] / r if adjusted[t] > 0 else adjusted[t] * r
    adjusted = adjusted / np.float32(temperature)
    e = np.exp((adjusted - adjusted.max()).astype(np.float32)).astype(np.float32)
    probs = e / e.sum(dtype=np.float32)
    order = sorted(range(probs.size), key=lambda i: (-float(probs[i]), i))
    order = order[: min(top_k, probs.size)]
    cumulative = np.float32(0)
    cutoff = len(order)
    for n, i in enumerate(order):
        cumulative += probs[i]
        if cumulative >= np.float32(top_p):
            cutoff = n + 1
            break
    order = order[:cutoff]
    return order, [float(probs[i]) for i in order]
