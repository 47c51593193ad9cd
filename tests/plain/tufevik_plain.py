"""Plain, slow, whole-sequence implementation of the Tufevik decoder.

The oracle of the Tufevik tests: no cache, no batching, no kernels, one function per mechanism, float64 torch ops on
the CPU.  It shares no code with the engine package: it reads ``config.json`` and the safetensors file by itself and
takes every size and constant from the configuration dictionary.

Notation: T tokens, W the model width, x [T, W].  Linear weights are kept [out, in] and applied as x @ W^T.

The design
* embeds a token as table[token] * embedding.scale and ties the output head to the table (without the scale);
* wraps every sublayer in two norms: x <- x + after(sublayer(before(x)));
* norms with a tanh instead of statistics: tanh(alpha x) * w + b;
* has two token mixers: ``mlstm``, a matrix memory with exponential gates and a running maximum, and ``parallel``,
  the weighted sum of a grouped-query attention (short convolutions on q, k, v, one norm over all of q and over all
  of k, partly rotated heads with stretched frequencies, a gate per head) and a selective state-space scan;
* feeds forward densely (relu-gated) or through a mixture of experts whose weights are the softmax over the chosen
  logits.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- small parts
def tanh_norm(x: torch.Tensor, w: dict, name: str) -> torch.Tensor:
    """tanh(alpha x) * weight + bias; no mean, no variance."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """u [T, C], taps [C, K]: y_t = sum_j taps[:, j] u_(t - K + 1 + j), zeros before the sequence."""
    count, width = u.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(width - 1, u.shape[1], dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(width):
        y = y + padded[j:j + count] * taps[:, j]
    return y if bias is None else y + bias


# --------------------------------------------------------------------------- matrix memory
def capped(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def mlstm_gates(h: torch.Tensor, w: dict, prefix: str, cap: float):
    """Log input gate and log forget gate, [T, heads] each."""
    i = capped(h @ w[prefix + "i"].t() + w[prefix + "i.b"], cap)
    f = F.logsigmoid(capped(h @ w[prefix + "f"].t() + w[prefix + "f.b"], cap))
    return i, f


def mlstm_recurrence(q, k, v, i, f):
    """q, k [T, heads, d], v [T, heads, e], gates [T, heads] -> outputs [T, heads, e].  Token by token from a zero
    memory, a zero normaliser and a running maximum that starts at zero."""
    count, heads, d = q.shape
    e = v.shape[2]
    memory = torch.zeros(heads, d, e, dtype=q.dtype)
    normaliser = torch.zeros(heads, d, dtype=q.dtype)
    m = torch.zeros(heads, dtype=q.dtype)
    out = []
    for t in range(count):
        m_new = torch.maximum(f[t] + m, i[t])
        keep = torch.exp(f[t] + m - m_new)
        take = torch.exp(i[t] - m_new)
        memory = keep[:, None, None] * memory + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        normaliser = keep[:, None] * normaliser + take[:, None] * k[t]
        m = m_new
        read = torch.einsum("hde,hd->he", memory, q[t])
        weight = (normaliser * q[t]).sum(-1).abs()
        out.append(read / (torch.maximum(weight, torch.exp(-m)) + 1e-6)[:, None])
    return torch.stack(out)


def mlstm(h: torch.Tensor, w: dict, prefix: str, mixer: dict, eps: float) -> torch.Tensor:
    heads, d, e = int(mixer["heads"]), int(mixer["dim"]), int(mixer["vdim"])
    count = h.shape[0]
    q = (h @ w[prefix + "q"].t()).view(count, heads, d) * d ** -0.5
    k = (h @ w[prefix + "k"].t()).view(count, heads, d)
    v = (h @ w[prefix + "v"].t()).view(count, heads, e)
    i, f = mlstm_gates(h, w, prefix, float(mixer["gate_cap"]))
    read = rms(mlstm_recurrence(q, k, v, i, f), eps).reshape(count, heads * e)
    return (read * w[prefix + "norm"] * torch.sigmoid(h @ w[prefix + "g"].t())) @ w[prefix + "o"].t()


# --------------------------------------------------------------------------- attention side
def rotary_table(rot: dict, count: int, first: int = 0):
    """cos, sin [T, dims / 2] of positions first .. first + T - 1, with the stretched frequencies when ``scaling``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    index = torch.arange(dims // 2, dtype=torch.float64)
    freq = base ** (-2.0 * index / dims)
    factor = 1.0
    scaling = rot.get("scaling")
    if scaling:
        s, original = float(scaling["factor"]), float(scaling["original"])

        def turns_index(turns: float) -> float:
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(turns_index(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turns_index(float(scaling["slow"]))), dims - 1)
        ramp = ((index - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        freq = freq / s * ramp + freq * (1.0 - ramp)
        factor = 0.1 * math.log(s) + 1.0
    angle = torch.arange(first, first + count, dtype=torch.float64)[:, None] * freq[None, :]
    return torch.cos(angle) * factor, torch.sin(angle) * factor


def rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, dims: int) -> torch.Tensor:
    """x [T, heads, d]: dimension i is paired with i + dims / 2 for i < dims / 2; the rest passes."""
    half = dims // 2
    a, b, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)


def causal_softmax_attention(q, k, v, scale: float) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e]; row i sees columns j <= i."""
    heads, groups = q.shape[1], k.shape[1]
    k = k.repeat_interleave(heads // groups, dim=1)
    v = v.repeat_interleave(heads // groups, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    count = q.shape[0]
    scores = scores.masked_fill(torch.ones(count, count, dtype=torch.bool).triu(1), float("-inf"))
    return torch.einsum("hij,jhe->ihe", torch.softmax(scores, dim=-1), v)


def conv_attention(h: torch.Tensor, w: dict, prefix: str, m: dict, eps: float) -> torch.Tensor:
    heads, groups, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    count = h.shape[0]
    q = causal_conv(h @ w[prefix + "q"].t(), w[prefix + "q.conv"])
    k = causal_conv(h @ w[prefix + "k"].t(), w[prefix + "k.conv"])
    v = causal_conv(h @ w[prefix + "v"].t(), w[prefix + "v.conv"])
    q = rms(q, eps) * w[prefix + "q.norm"]          # one norm over the whole projection, before the heads are cut
    k = rms(k, eps) * w[prefix + "k.norm"]
    cos, sin = rotary_table(m["rot"], count)
    dims = int(m["rot"]["dims"])
    q = rotate_half(q.view(count, heads, d), cos, sin, dims)
    k = rotate_half(k.view(count, groups, d), cos, sin, dims)
    out = causal_softmax_attention(q, k, v.view(count, groups, e), float(m["scale"]))
    out = out * torch.sigmoid(h @ w[prefix + "g"].t())[:, :, None]      # one gate per head
    return out.reshape(count, heads * e) @ w[prefix + "o"].t()


# --------------------------------------------------------------------------- state-space side
def selective_scan(x, dt, a, b, c, skip) -> torch.Tensor:
    """x, dt [T, C]; a [C, N]; b, c [T, N]; skip [C]:  S <- exp(dt a) S + dt x b;  y = S c + skip x."""
    state = torch.zeros_like(a)
    out = []
    for t in range(x.shape[0]):
        state = torch.exp(dt[t][:, None] * a) * state + (dt[t] * x[t])[:, None] * b[t][None, :]
        out.append(state @ c[t] + skip * x[t])
    return torch.stack(out)


def state_space(h: torch.Tensor, w: dict, prefix: str, m: dict) -> torch.Tensor:
    inner, rank, states = int(m["inner"]), int(m["dt_rank"]), int(m["state"])
    xz = h @ w[prefix + "in"].t()
    x, z = xz[:, :inner], xz[:, inner:]
    x = F.silu(causal_conv(x, w[prefix + "conv"], w[prefix + "conv.b"]))
    low = x @ w[prefix + "x"].t()
    dt = F.softplus(low[:, :rank] @ w[prefix + "dt"].t() + w[prefix + "dt.b"])
    b, c = low[:, rank:rank + states], low[:, rank + states:]
    y = selective_scan(x, dt, -torch.exp(w[prefix + "A_log"]), b, c, w[prefix + "D"])
    return (y * F.silu(z)) @ w[prefix + "o"].t()


def parallel(h: torch.Tensor, w: dict, prefix: str, mixer: dict, eps: float) -> torch.Tensor:
    left = conv_attention(h, w, prefix + "left.", mixer["left"], eps)
    right = state_space(h, w, prefix + "right.", mixer["right"])
    return float(mixer["left_scale"]) * left + float(mixer["right_scale"]) * right


# --------------------------------------------------------------------------- feed-forward
def dense(h: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    return (torch.relu(h @ w[prefix + "gate"].t()) * (h @ w[prefix + "up"].t())) @ w[prefix + "down"].t()


def route(h: torch.Tensor, w: dict, prefix: str, top: int):
    """(chosen [T, top], weights [T, top]): the largest logits, softmax over the chosen logits only."""
    logits = h @ w[prefix + "router"].t() + w[prefix + "router.b"]
    values, chosen = torch.topk(logits, top, dim=-1)
    return chosen, torch.softmax(values, dim=-1)


def mixture(h: torch.Tensor, w: dict, prefix: str, mlp: dict) -> torch.Tensor:
    chosen, weights = route(h, w, prefix, int(mlp["router"]["top"]))
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, share in zip(chosen[t].tolist(), weights[t]):
            name = f"{prefix}e{e}."
            row = h[t]
            y[t] += share * ((F.silu(w[name + "gate"] @ row) * (w[name + "up"] @ row)) @ w[name + "down"].t())
    return y


# --------------------------------------------------------------------------- the model
def forward_layers(cfg: dict, w: dict, tokens: list[int]) -> list[torch.Tensor]:
    """The residual after the embedding and after every layer: a list of [T, W]."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    seen = [x]
    for index, layer in enumerate(cfg["layers"]):
        p = f"l{index}."
        h = tanh_norm(x, w, p + "norm1")
        if layer["type"] == "mlstm":
            y = mlstm(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + tanh_norm(y, w, p + "norm1b")
        mlp = layer.get("mlp")
        if mlp is not None:
            h = tanh_norm(x, w, p + "norm2")
            y = dense(h, w, p + "mlp.") if mlp["kind"] == "dense" else mixture(h, w, p + "mlp.", mlp)
            x = x + tanh_norm(y, w, p + "norm2b")
        seen.append(x)
    return seen


def logits_of(cfg: dict, w: dict, x: torch.Tensor) -> torch.Tensor:
    return tanh_norm(x, w, "final.norm") @ w["embed"].t()


def forward_full(cfg: dict, w: dict, tokens: list[int]) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence."""
    return logits_of(cfg, w, forward_layers(cfg, w, tokens)[-1])


# --------------------------------------------------------------------------- files
_STORED = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """The file format read directly: an 8-byte little-endian length, that many bytes of JSON (name -> dtype, shape,
    data_offsets), then the data."""
    raw = Path(path).read_bytes()
    (length,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + length])
    data = raw[8 + length:]
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        lo, hi = entry["data_offsets"]
        tensor = torch.frombuffer(bytearray(data[lo:hi]), dtype=_STORED[entry["dtype"]])
        out[name] = tensor.reshape(entry["shape"])
    return out


def load_folder(folder, round_to=None):
    """(config dictionary, weights in float64).  ``round_to`` (e.g. torch.bfloat16): matrices are rounded to it first,
    as an engine that holds them so would see them."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = {}
    for name, tensor in read_safetensors(folder / "model.safetensors").items():
        if tensor.is_floating_point():
            if round_to is not None and tensor.dim() >= 2:
                tensor = tensor.to(round_to)
            tensor = tensor.to(torch.float64)
        weights[name] = tensor
    return cfg, weights


# --------------------------------------------------------------------------- random models for the tests
def tensor_shapes(cfg: dict) -> dict[str, tuple]:
    """Every tensor of a model of this configuration, by name."""
    width = int(cfg["width"])
    shapes = {"embed": (int(cfg["vocab"]), width)}

    def tanh_norm_shapes(name: str) -> None:
        shapes[name], shapes[name + ".b"], shapes[name + ".alpha"] = (width,), (width,), ()

    for index, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{index}."
        for name in ("norm1", "norm1b") + (("norm2", "norm2b") if layer.get("mlp") is not None else ()):
            tanh_norm_shapes(p + name)
        if layer["type"] == "mlstm":
            heads, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            shapes.update({p + "mix.q": (heads * d, width), p + "mix.k": (heads * d, width), p + "mix.v": (heads * e, width),
                           p + "mix.g": (heads * e, width), p + "mix.o": (width, heads * e), p + "mix.norm": (heads * e,),
                           p + "mix.i": (heads, width), p + "mix.i.b": (heads,), p + "mix.f": (heads, width),
                           p + "mix.f.b": (heads,)})
        else:
            left, right = m["left"], m["right"]
            heads, groups, d, e, taps = (int(left[key]) for key in ("heads", "kv_heads", "dim", "vdim", "conv"))
            a = p + "mix.left."
            shapes.update({a + "q": (heads * d, width), a + "k": (groups * d, width), a + "v": (groups * e, width),
                           a + "q.norm": (heads * d,), a + "k.norm": (groups * d,), a + "q.conv": (heads * d, taps),
                           a + "k.conv": (groups * d, taps), a + "v.conv": (groups * e, taps), a + "g": (heads, width),
                           a + "o": (width, heads * e)})
            inner, rank, states, taps = (int(right[key]) for key in ("inner", "dt_rank", "state", "conv"))
            b = p + "mix.right."
            shapes.update({b + "in": (2 * inner, width), b + "conv": (inner, taps), b + "conv.b": (inner,),
                           b + "x": (rank + 2 * states, inner), b + "dt": (inner, rank), b + "dt.b": (inner,),
                           b + "A_log": (inner, states), b + "D": (inner,), b + "o": (width, inner)})
        mlp = layer.get("mlp")
        if mlp is not None and mlp["kind"] == "dense":
            ff = int(mlp["ff"])
            shapes.update({p + "mlp.gate": (ff, width), p + "mlp.up": (ff, width), p + "mlp.down": (width, ff)})
        elif mlp is not None:
            experts, ff = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            shapes[p + "mlp.router"], shapes[p + "mlp.router.b"] = (experts, width), (experts,)
            for j in range(experts):
                shapes.update({f"{p}mlp.e{j}.gate": (ff, width), f"{p}mlp.e{j}.up": (ff, width),
                               f"{p}mlp.e{j}.down": (width, ff)})
    tanh_norm_shapes("final.norm")
    return shapes


def random_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random float32 weights with gains large enough that every mechanism moves the logits: gates that open and
    close, a memory whose maximum moves, routers with clear choices, step sizes and decays of the scan spread over
    a range."""
    generator = torch.Generator().manual_seed(seed)

    def normal(shape, std):
        return torch.randn(shape, generator=generator) * std

    def uniform(shape, lo, hi):
        return lo + (hi - lo) * torch.rand(shape, generator=generator)

    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        before = name.rsplit(".", 2)[-2] if name.count(".") >= 2 else ""
        if name == "embed":
            tensor = normal(shape, 0.08)
        elif last == "alpha":
            tensor = uniform(shape, 0.4, 1.2)
        elif last == "A_log":
            tensor = torch.log(uniform(shape, 0.3, 4.0))
        elif last == "D":
            tensor = uniform(shape, 0.5, 1.5)
        elif last == "conv":
            tensor = normal(shape, 0.5)
        elif last == "b" and before == "dt":
            tensor = torch.log(torch.expm1(uniform(shape, 0.01, 0.3)))       # softplus^-1 of a step size
        elif last == "b" and before in ("i", "f"):
            tensor = normal(shape, 1.0) + (2.0 if before == "f" else 0.0)
        elif last == "b":
            tensor = normal(shape, 0.2)
        elif last in ("norm", "norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            tensor = uniform(shape, 0.6, 1.4)
        elif last in ("i", "f"):
            tensor = normal(shape, 3.0 / shape[1] ** 0.5)
        elif last == "router":
            tensor = normal(shape, 4.0 / shape[1] ** 0.5)
        elif last == "dt":
            tensor = normal(shape, 1.0 / shape[1] ** 0.5)
        elif last in ("gate", "up", "q", "k"):
            tensor = normal(shape, 1.5 / shape[1] ** 0.5)
        else:
            tensor = normal(shape, 1.0 / shape[1] ** 0.5)
        out[name] = tensor.to(torch.bfloat16).to(torch.float32).contiguous()   # values that bfloat16 holds exactly
    return out


def write_model(folder, cfg: dict, seed: int, weights: dict | None = None) -> dict[str, torch.Tensor]:
    """config.json and model.safetensors (float32) of a random model (or of ``weights``); returns the weights."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    weights = weights if weights is not None else random_weights(cfg, seed)
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    save_file({name: tensor.contiguous() for name, tensor in weights.items()}, str(folder / "model.safetensors"))
    return weights
