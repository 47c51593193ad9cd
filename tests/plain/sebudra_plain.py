"""Plain, slow, whole-sequence implementation of the Sebudra decoder.

The oracle of the Sebudra tests: no cache, no batching, no kernels, one function per mechanism, float64 torch ops on
the CPU.  It shares no code with the engine package: it reads ``config.json`` and the safetensors file by itself and
takes every size and constant from the configuration dictionary.

Notation: T tokens, W the model width, x [T, W].  Linear weights are kept [out, in] and applied as x @ W^T.

The design
* embeds a token as table[token] * embedding.scale and has a head matrix of its own;
* runs both sublayers of a layer on ONE normed input: n = rmsnorm(x), x <- x + mixer(n) + feed_forward(n);
* has three token mixers: ``parallel`` (the weighted sum of a sliding-window softmax attention with biases, normed
  and partly rotated heads with stretched frequencies, and a state-space scan with one decay per head and token),
  ``attention`` (causal, capped scores, every key weighted by a sigmoid of its own score, no normalisation) and
  ``gla`` (a matrix memory whose rows decay by a learned factor per key channel and token);
* feeds forward densely (clamped, swish-gated) or through a mixture of squared-relu experts chosen among the best
  groups of experts by sigmoid scores, with a gated shared expert;
* lets a layer run with another layer's tensors (``weights_of``).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- small parts
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K]: y_t = bias + sum_j taps[:, j] u_(t - K + 1 + j), zeros before the sequence."""
    count, width = u.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(width - 1, u.shape[1], dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(width):
        y = y + padded[j:j + count] * taps[:, j]
    return y + bias


# --------------------------------------------------------------------------- rotation
def rotary_table(rot: dict, count: int):
    """cos, sin [count, dims / 2] of the angles position * frequency_i, frequency_i = base^(-2i / dims); with
    ``scaling`` the low frequencies are divided by ``factor`` along a ramp and both tables grow by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    grow = 1.0
    scaling = rot.get("scaling")
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def turn_dim(turns: float) -> float:
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
        ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=torch.float64)
        freq = freq / factor * ramp + freq * (1.0 - ramp)
        grow = 0.1 * math.log(factor) + 1.0
    angle = torch.arange(count, dtype=torch.float64)[:, None] * freq[None, :]
    return torch.cos(angle) * grow, torch.sin(angle) * grow


def rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, dims: int) -> torch.Tensor:
    """x [T, heads, d]: value i of the first ``dims`` is paired with value i + dims / 2; the rest pass."""
    half = dims // 2
    a, b, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)


def normed_rotated_heads(h, w, prefix, m, eps, bias: bool):
    """q [T, H, d], k [T, G, d], v [T, G, e]: projections (with biases when ``bias``), an RMS norm over each head of q
    and k with one weight vector for all heads, then the rotation of q and k."""
    count = h.shape[0]
    heads, groups, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])

    def project(name):
        y = h @ w[prefix + name].t()
        return y + w[prefix + name + ".b"] if bias else y

    q = rms(project("q").view(count, heads, d), eps) * w[prefix + "q.norm"]
    k = rms(project("k").view(count, groups, d), eps) * w[prefix + "k.norm"]
    v = project("v").view(count, groups, e)
    rot = m.get("rot")
    if rot and int(rot["dims"]) > 0:
        cos, sin = rotary_table(rot, count)
        q, k = rotate_half(q, cos, sin, int(rot["dims"])), rotate_half(k, cos, sin, int(rot["dims"]))
    return q, k, v


def key_scores(q, k, scale: float) -> torch.Tensor:
    """[H, T, T] scores of every query head against the keys of its group."""
    heads, groups = q.shape[1], k.shape[1]
    k = k.repeat_interleave(heads // groups, dim=1)
    return torch.einsum("ihd,jhd->hij", q, k) * scale


def apply_weights(weights: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """weights [H, T, T], v [T, G, e] -> [T, H * e]."""
    heads = weights.shape[0]
    v = v.repeat_interleave(heads // v.shape[1], dim=1)
    return torch.einsum("hij,jhe->ihe", weights, v).reshape(v.shape[0], -1)


# --------------------------------------------------------------------------- the three mixers
def window_attention(h, w, prefix, m, eps) -> torch.Tensor:
    """Softmax attention in which row i sees rows j with 0 <= i - j < mask.size; [T, H * e] before the output matrix."""
    q, k, v = normed_rotated_heads(h, w, prefix, m, eps, bias=True)
    count = h.shape[0]
    scores = key_scores(q, k, float(m["scale"]))
    distance = torch.arange(count)[:, None] - torch.arange(count)[None, :]
    seen = (distance >= 0) & (distance < int(m["mask"]["size"]))
    scores = scores.masked_fill(~seen, float("-inf"))
    return apply_weights(torch.softmax(scores, dim=-1), v)


def state_space_scan(x, dt, decay_rate, b, c, skip) -> torch.Tensor:
    """x [T, H, e], dt [T, H], decay_rate [H], b and c [T, H, N] (already spread from groups to heads), skip [H]:
    S <- exp(-decay_rate dt) S + dt b x^T;  y = S^T c + skip x.  S [H, N, e] starts at zero."""
    count, heads, e = x.shape
    state = torch.zeros(heads, b.shape[2], e, dtype=x.dtype)
    out = []
    for t in range(count):
        keep = torch.exp(-decay_rate * dt[t])
        state = keep[:, None, None] * state + dt[t][:, None, None] * b[t][:, :, None] * x[t][:, None, :]
        out.append(torch.einsum("hne,hn->he", state, c[t]) + skip[:, None] * x[t])
    return torch.stack(out)


def state_space(h, w, prefix, m, eps) -> torch.Tensor:
    """The scan side of a ``parallel`` mixer; [T, heads * vdim] before the output matrix."""
    count = h.shape[0]
    heads, e, n, groups = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = heads * e
    proj = h @ w[prefix + "in"].t()
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * groups * n], proj[:, 2 * inner + 2 * groups * n:]
    xbc = F.silu(causal_conv(xbc, w[prefix + "conv"], w[prefix + "conv.b"]))
    x = xbc[:, :inner].view(count, heads, e)
    b = xbc[:, inner:inner + groups * n].view(count, groups, n).repeat_interleave(heads // groups, dim=1)
    c = xbc[:, inner + groups * n:].view(count, groups, n).repeat_interleave(heads // groups, dim=1)
    dt = F.softplus(dt + w[prefix + "dt_bias"])
    y = state_space_scan(x, dt, torch.exp(w[prefix + "A_log"]), b, c, w[prefix + "D"]).reshape(count, inner)
    y = y * F.silu(z)
    parts = int(m["norm_groups"])
    y = rms(y.view(count, parts, inner // parts), eps).reshape(count, inner)
    return y * w[prefix + "norm"]


def parallel_mixer(h, w, prefix, mixer, eps) -> torch.Tensor:
    left = window_attention(h, w, prefix + "left.", mixer["left"], eps) @ w[prefix + "left.o"].t()
    right = state_space(h, w, prefix + "right.", mixer["right"], eps) @ w[prefix + "right.o"].t()
    return float(mixer["left_scale"]) * left + float(mixer["right_scale"]) * right


def sigmoid_attention(h, w, prefix, m, eps) -> torch.Tensor:
    """Causal attention whose weights are sigmoid(capped score + a number per head), not normalised over the keys."""
    q, k, v = normed_rotated_heads(h, w, prefix, m, eps, bias=False)
    count = h.shape[0]
    scores = key_scores(q, k, float(m["scale"]))
    cap = float(m["softcap"])
    scores = cap * torch.tanh(scores / cap)
    weights = torch.sigmoid(scores + w[prefix + "pb"][:, None, None])
    seen = torch.arange(count)[:, None] >= torch.arange(count)[None, :]
    weights = weights * seen
    return apply_weights(weights, v) @ w[prefix + "o"].t()


def decayed_memory(q, k, v, keep) -> torch.Tensor:
    """q, k, keep [T, H, d], v [T, H, e]:  S <- diag(keep_t) S + k_t v_t^T;  o_t = S^T q_t.  S [H, d, e] from zero."""
    count, heads, d = q.shape
    state = torch.zeros(heads, d, v.shape[2], dtype=q.dtype)
    out = []
    for t in range(count):
        state = keep[t][:, :, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hde,hd->he", state, q[t]))
    return torch.stack(out)


def gla(h, w, prefix, m, eps) -> torch.Tensor:
    count = h.shape[0]
    heads, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[prefix + "q"].t()).view(count, heads, d) * d ** -0.5
    k = (h @ w[prefix + "k"].t()).view(count, heads, d)
    v = (h @ w[prefix + "v"].t()).view(count, heads, e)
    z = (h @ w[prefix + "a1"].t()) @ w[prefix + "a2"].t() + w[prefix + "a2.b"]
    keep = torch.exp(F.logsigmoid(z) / float(m["tau"])).view(count, heads, d)
    o = rms(decayed_memory(q, k, v, keep), eps) * w[prefix + "norm"]
    return (o.reshape(count, heads * e) * F.silu(h @ w[prefix + "g"].t())) @ w[prefix + "o"].t()


# --------------------------------------------------------------------------- feed-forwards
def dense(h, w, prefix, mlp) -> torch.Tensor:
    limit = float(mlp["limit"])
    g = (h @ w[prefix + "gate"].t()).clamp(max=limit)
    u = (h @ w[prefix + "up"].t()).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[prefix + "down"].t()


def squared_relu_expert(h, w, prefix) -> torch.Tensor:
    return F.relu(h @ w[prefix + "up"].t()).pow(2) @ w[prefix + "down"].t()


def route(h, w, prefix, router: dict):
    """(chosen [T, top], weights [T, top]).  Scores are sigmoids of the router's logits; the choice adds the
    correction and is confined to the ``keep`` groups of neighbouring experts whose two best choice scores sum highest;
    the weights are the chosen plain scores over their sum, times ``scale``."""
    experts, top = int(router["experts"]), int(router["top"])
    scores = torch.sigmoid(h @ w[prefix + "router"].t())
    choice = scores + w[prefix + "correction"]
    groups = router.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = experts // count
        grouped = choice.view(-1, count, per)
        group_score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
        best = group_score.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, best, True)
        choice = grouped.masked_fill(~allowed[:, :, None], float("-inf")).reshape(-1, experts)
    chosen = choice.topk(top, dim=-1).indices
    picked = scores.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20) * float(router["scale"])


def mixture(h, w, prefix, mlp) -> torch.Tensor:
    chosen, weights = route(h, w, prefix, mlp["router"])
    y = torch.zeros_like(h)
    for e in range(int(mlp["router"]["experts"])):
        share = (weights * (chosen == e)).sum(-1, keepdim=True)
        if bool((share != 0).any()):
            y = y + share * squared_relu_expert(h, w, f"{prefix}e{e}.")
    if mlp.get("shared"):
        y = y + torch.sigmoid(h @ w[prefix + "shared.sg"].t()) * squared_relu_expert(h, w, prefix + "shared.")
    return y


# --------------------------------------------------------------------------- the model
def layer_prefix(cfg: dict, index: int) -> str:
    source = cfg["layers"][index].get("weights_of")
    return f"l{index if source is None else int(source)}."


def forward_layers(cfg: dict, w: dict, tokens: list[int]) -> list[torch.Tensor]:
    """The residual after the embedding and after every layer run: a list of [T, W]."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    seen = [x]
    for index, layer in enumerate(cfg["layers"]):
        p = layer_prefix(cfg, index)
        n = rms(x, eps) * w[p + "norm1"]
        kind, mixer = layer["type"], layer["mixer"]
        if kind == "parallel":
            y = parallel_mixer(n, w, p + "mix.", mixer, eps)
        elif kind == "attention":
            y = sigmoid_attention(n, w, p + "mix.", mixer, eps)
        elif kind == "gla":
            y = gla(n, w, p + "mix.", mixer, eps)
        else:
            raise ValueError(f"layer {index}: unknown type {kind!r}")
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + (dense(n, w, p + "mlp.", mlp) if mlp["kind"] == "dense" else mixture(n, w, p + "mlp.", mlp))
        x = x + y
        seen.append(x)
    return seen


def logits_of(cfg: dict, w: dict, x: torch.Tensor) -> torch.Tensor:
    return (rms(x, float(cfg["norm"]["eps"])) * w["final.norm"]) @ w["head"].t()


def forward_full(cfg: dict, w: dict, tokens: list[int]) -> torch.Tensor:
    """Logits [T, vocab] at every position of one sequence."""
    return logits_of(cfg, w, forward_layers(cfg, w, tokens)[-1])


# --------------------------------------------------------------------------- files
_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    raw = Path(path).read_bytes()
    (length,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + length])
    data = raw[8 + length:]
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        lo, hi = entry["data_offsets"]
        tensor = torch.frombuffer(bytearray(data[lo:hi]), dtype=_DTYPES[entry["dtype"]]).reshape(entry["shape"])
        out[name] = tensor
    return out


def load_folder(folder, round_to=None):
    """(config dictionary, weights in float64).  ``round_to``: round the weights to this dtype first."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = {}
    for name, tensor in read_safetensors(folder / "model.safetensors").items():
        if tensor.is_floating_point():
            tensor = (tensor.to(round_to) if round_to is not None else tensor).to(torch.float64)
        weights[name] = tensor
    return cfg, weights


def tensor_shapes(cfg: dict) -> dict[str, tuple]:
    """name -> (shape, kind) of every tensor of a model of this configuration; kind says how random values are drawn."""
    width, vocab = int(cfg["width"]), int(cfg["vocab"])
    out = {"embed": ((vocab, width), "matrix"), "final.norm": ((width,), "norm"), "head": ((vocab, width), "matrix")}
    for index, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p = f"l{index}."
        out[p + "norm1"] = ((width,), "norm")
        kind, m = layer["type"], layer["mixer"]
        if kind in ("parallel", "attention"):
            a, q = (m["left"], p + "mix.left.") if kind == "parallel" else (m, p + "mix.")
            heads, groups, d, e = int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"])
            for name, rows in (("q", heads * d), ("k", groups * d), ("v", groups * e)):
                out[q + name] = ((rows, width), "matrix")
                if kind == "parallel":
                    out[q + name + ".b"] = ((rows,), "bias")
            out[q + "q.norm"] = ((d,), "norm")
            out[q + "k.norm"] = ((d,), "norm")
            out[q + "o"] = ((width, heads * e), "matrix")
            if kind == "attention":
                out[q + "pb"] = ((heads,), "head_bias")
        if kind == "parallel":
            r, q = m["right"], p + "mix.right."
            heads, e, n, groups, taps = int(r["heads"]), int(r["vdim"]), int(r["state"]), int(r["groups"]), int(r["conv"])
            inner, channels = heads * e, heads * e + 2 * groups * n
            out[q + "in"] = ((2 * inner + 2 * groups * n + heads, width), "matrix")
            out[q + "conv"] = ((channels, taps), "filter")
            out[q + "conv.b"] = ((channels,), "bias")
            out[q + "dt_bias"] = ((heads,), "bias")
            out[q + "A_log"] = ((heads,), "bias")
            out[q + "D"] = ((heads,), "norm")
            out[q + "norm"] = ((inner,), "norm")
            out[q + "o"] = ((width, inner), "matrix")
        if kind == "gla":
            q = p + "mix."
            heads, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            rank = int(m["rank"])       # no key of the design's own: a model written here names it
            out[q + "q"] = ((heads * d, width), "matrix")
            out[q + "k"] = ((heads * d, width), "matrix")
            out[q + "v"] = ((heads * e, width), "matrix")
            out[q + "g"] = ((heads * e, width), "matrix")
            out[q + "o"] = ((width, heads * e), "matrix")
            out[q + "norm"] = ((e,), "norm")
            out[q + "a1"] = ((rank, width), "matrix")
            out[q + "a2"] = ((heads * d, rank), "wide_matrix")
            out[q + "a2.b"] = ((heads * d,), "decay_bias")
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        q = p + "mlp."
        if mlp["kind"] == "dense":
            ff = int(mlp["ff"])
            out[q + "gate"] = ((ff, width), "matrix")
            out[q + "up"] = ((ff, width), "matrix")
            out[q + "down"] = ((width, ff), "matrix")
        else:
            experts, ff = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            for e in range(experts):
                out[f"{q}e{e}.up"] = ((ff, width), "matrix")
                out[f"{q}e{e}.down"] = ((width, ff), "matrix")
            out[q + "router"] = ((experts, width), "matrix")
            out[q + "correction"] = ((experts,), "bias")
            if mlp.get("shared"):
                ff = int(mlp["shared"]["ff"])
                out[q + "shared.up"] = ((ff, width), "matrix")
                out[q + "shared.down"] = ((width, ff), "matrix")
                out[q + "shared.sg"] = ((1, width), "matrix")
    return out


def random_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random weights, rounded to bfloat16 values: large enough that every mechanism moves the logits."""
    generator = torch.Generator().manual_seed(seed)
    width = int(cfg["width"])
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        if kind == "matrix":
            t = torch.randn(shape, generator=generator) * (1.0 / math.sqrt(shape[-1]))
            if name == "embed":
                t = torch.randn(shape, generator=generator) * 0.5
        elif kind == "wide_matrix":
            t = torch.randn(shape, generator=generator) * (2.0 / math.sqrt(shape[-1]))
        elif kind == "norm":
            t = 1.0 + 0.2 * (torch.rand(shape, generator=generator) - 0.5)
        elif kind == "bias":
            t = 0.3 * torch.randn(shape, generator=generator)
        elif kind == "head_bias":
            t = -2.0 + 0.5 * torch.randn(shape, generator=generator)
        elif kind == "decay_bias":
            t = 2.0 + torch.randn(shape, generator=generator)
        elif kind == "filter":
            t = torch.randn(shape, generator=generator) * 0.5
        else:
            raise ValueError(kind)
        out[name] = t.to(torch.bfloat16)
    del width
    return out


def write_safetensors(path, tensors: dict[str, torch.Tensor]) -> None:
    names = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32"}
    header, blobs, offset = {}, [], 0
    for name, tensor in tensors.items():
        tensor = tensor.contiguous()
        blob = tensor.view(torch.uint8).numpy().tobytes() if tensor.numel() else b""
        header[name] = {"dtype": names[tensor.dtype], "shape": list(tensor.shape), "data_offsets": [offset, offset + len(blob)]}
        blobs.append(blob)
        offset += len(blob)
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)))
        handle.write(text)
        for blob in blobs:
            handle.write(blob)


def write_model(folder, cfg: dict, seed: int, weights: dict | None = None) -> dict[str, torch.Tensor]:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    weights = weights if weights is not None else random_weights(cfg, seed)
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(folder / "model.safetensors", weights)
    return weights
