"""Plain, slow implementation of the Lodalix decoder: one function per mechanism, float64 on the
CPU, token by token where the design is recurrent.  It shares no code with the engine; the GPU
tests hold the engine to it.

Notation: ``h`` is a sublayer's input [T, width]; a weight ``W`` is stored [out, in] and applied as
``h @ W.T``; ``p`` maps a layer's tensor names (without the layer prefix) to float64 tensors;
``first`` is the position of the first row of ``h`` in its request.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_gain_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight lies around zero: the gain is 1 + w."""
    return rms_divide(x, eps) * (1.0 + w)


def plain_gain_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_divide(x, eps) * w


def rotary_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """Frequencies f_i (i < dims/2) and the factor both cos and sin are multiplied with.  With a
    ``scaling`` entry the frequencies are blended between f_i and f_i / factor over a ramp whose
    ends are the pair indices at which ``original`` positions make ``fast`` and ``slow`` turns."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=F)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict, pairing: str) -> torch.Tensor:
    """x [T, ..., dims]: pair (u, v) at position p and frequency f becomes
    (u cos pf - v sin pf, v cos pf + u sin pf), both times the magnitude factor.  ``pairing``
    "interleaved": (2i, 2i+1); "half": (i, i + dims/2)."""
    f, magnitude = rotary_frequencies(rot)
    dims = int(rot["dims"])
    half = dims // 2
    angle = positions.to(F).view(-1, *([1] * (x.dim() - 2)), 1) * f
    cos, sin = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    out = x.clone()
    if pairing == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    return out


def latent_keys(h: torch.Tensor, p: dict, mixer: dict, eps: float, first: int, pairing: str):
    """What a latent-attention layer caches for the rows of ``h``: the normalised latent
    [T, kv_rank] and the rotated key part shared by all heads [T, rot_dim]."""
    rank = mixer["kv_rank"]
    down = h @ p["mix.dkv"].T
    latent = plain_gain_norm(down[:, :rank], p["mix.dkv.norm"], eps)
    positions = torch.arange(first, first + h.shape[0])
    return latent, rotate(down[:, rank:], positions, mixer["rot"], pairing)


def latent_attention(h: torch.Tensor, p: dict, mixer: dict, eps: float, first: int, pairing: str,
                     latent: torch.Tensor, shared_key: torch.Tensor, sink: bool, gate: bool) -> torch.Tensor:
    """Causal attention whose keys and values are expanded from a cached latent.  ``latent`` and
    ``shared_key`` hold positions 0 .. first + T - 1.  Head j: query = [dim plain, rot_dim rotated],
    key = [W_uk latent, shared rotated part], value = W_uv latent.  ``sink``: the softmax
    denominator gets one more term exp(sink_j), without key, value or scale.  ``gate``: the heads
    side by side are multiplied by sigmoid(W_g h) before the output projection."""
    heads, dim, rot_dim, vdim = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"]
    tokens = h.shape[0]
    q_latent = plain_gain_norm(h @ p["mix.dq"].T, p["mix.dq.norm"], eps)
    q = (q_latent @ p["mix.uq"].T).view(tokens, heads, dim + rot_dim)
    positions = torch.arange(first, first + tokens)
    q_rot = rotate(q[..., dim:], positions, mixer["rot"], pairing)
    keys = (latent @ p["mix.uk"].T).view(-1, heads, dim)
    values = (latent @ p["mix.uv"].T).view(-1, heads, vdim)
    out = torch.zeros(tokens, heads, vdim, dtype=F)
    for t in range(tokens):
        seen = first + t + 1
        for j in range(heads):
            score = (keys[:seen, j] @ q[t, j, :dim] + shared_key[:seen] @ q_rot[t, j]) * mixer["scale"]
            top = score.max()
            if sink:
                top = torch.maximum(top, p["mix.sink"][j])
            weight = torch.exp(score - top)
            total = weight.sum()
            if sink:
                total = total + torch.exp(p["mix.sink"][j] - top)
            out[t, j] = (weight / total) @ values[:seen, j]
    flat = out.reshape(tokens, heads * vdim)
    if gate:
        flat = flat * torch.sigmoid(h @ p["mix.g"].T)
    return flat @ p["mix.o"].T


def delta_recurrence(r, k, v, w, a, state=None):
    """r, k, v, w, a: [T, heads, dim].  Per head, with u = k / sqrt(sum k^2 + 1e-6):
    S <- diag(w) S - (a * u) (u^T S) + k v^T (both first terms from the old S), o = S^T r.
    Returns o [T, heads, dim] and the last states [heads, dim, dim]."""
    tokens, heads, dim = r.shape
    out = torch.zeros(tokens, heads, dim, dtype=F)
    state = torch.zeros(heads, dim, dim, dtype=F) if state is None else state.clone().to(F)
    for t in range(tokens):
        for j in range(heads):
            unit = k[t, j] / torch.sqrt((k[t, j] ** 2).sum() + 1e-6)
            old = state[j]
            state[j] = w[t, j].unsqueeze(1) * old - torch.outer(a[t, j] * unit, unit @ old) + torch.outer(k[t, j], v[t, j])
            out[t, j] = state[j].T @ r[t, j]
    return out, state


def delta_mixer(h: torch.Tensor, p: dict, mixer: dict, eps: float, state=None):
    """Generalized delta rule with a decay and a removal rate per head and key channel."""
    heads, dim = mixer["heads"], mixer["dim"]
    tokens = h.shape[0]
    shape = (tokens, heads, dim)
    r, k, v = ((h @ p[f"mix.{n}"].T).view(shape) for n in "rkv")
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ p["mix.w1"].T) @ p["mix.w2"].T + p["mix.w0"]))
    removal = torch.sigmoid(h @ p["mix.a"].T + p["mix.a.b"])
    out, state = delta_recurrence(r, k, v, decay.view(shape), removal.view(shape), state)
    flat = rms_divide(out, eps).reshape(tokens, heads * dim) * p["mix.norm"]
    flat = flat * torch.sigmoid(h @ p["mix.g"].T)
    return flat @ p["mix.o"].T, state


def clamped_glu(h: torch.Tensor, p: dict, limit: float) -> torch.Tensor:
    """gate capped above, up clamped to both sides; gate * sigmoid(1.702 gate) * (up + 1)."""
    g = torch.clamp(h @ p["mlp.gate"].T + p["mlp.gate.b"], max=limit)
    u = torch.clamp(h @ p["mlp.up"].T + p["mlp.up.b"], -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ p["mlp.down"].T + p["mlp.down.b"]


PAIRING = {"latent_attention": "interleaved", "latent_attention_2": "half"}


def forward(config: dict, tensors: dict, tokens: list[int], layer_outputs: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one request run whole.  ``layer_outputs`` collects the residual stream
    after every layer."""
    t = {name: value.to(F) for name, value in tensors.items()}
    eps = config["norm"]["eps"]
    x = t["embed"][torch.tensor(tokens, dtype=torch.long)]
    caches: dict[int, tuple] = {}
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        p = {name[len(prefix):]: value for name, value in t.items() if name.startswith(prefix)}
        h = offset_gain_norm(x, p["norm1"], eps)
        kind, mixer = layer["type"], layer["mixer"]
        if kind in PAIRING:
            source = mixer.get("kv_from")
            if source is None:
                caches[index] = latent_keys(h, p, mixer, eps, 0, PAIRING[kind])
                source = index
            first_kind = kind == "latent_attention"
            y = latent_attention(h, p, mixer, eps, 0, PAIRING[kind], *caches[source],
                                 sink=first_kind, gate=not first_kind)
        elif kind == "general_delta":
            y, _ = delta_mixer(h, p, mixer, eps)
        else:
            raise ValueError(kind)
        if layer.get("mlp") is not None:
            y = y + clamped_glu(h, p, layer["mlp"]["limit"])
        x = x + y
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return offset_gain_norm(x, t["final.norm"], eps) @ t["head"].T


def first_token_delta_margin(config: dict, tensors: dict, tokens: list[int]) -> float:
    """At a request's first token a head of the delta rule puts out (k . r) v, and the head norm
    that follows keeps only the SIGN of k . r.  Returns the smallest |cos(k, r)| over all such heads:
    where it is nearly zero, rounding decides that sign and the row is no measure of anything."""
    t = {name: value.to(F) for name, value in tensors.items()}
    outputs: list = []
    forward(config, tensors, tokens[:1], outputs)
    inputs = [t["embed"][torch.tensor(tokens[:1], dtype=torch.long)]] + outputs
    margin = 1.0
    for index, layer in enumerate(config["layers"]):
        if layer["type"] != "general_delta":
            continue
        heads, dim = layer["mixer"]["heads"], layer["mixer"]["dim"]
        h = offset_gain_norm(inputs[index], t[f"l{index}.norm1"], config["norm"]["eps"])
        r = (h @ t[f"l{index}.mix.r"].T).view(heads, dim)
        k = (h @ t[f"l{index}.mix.k"].T).view(heads, dim)
        cosine = (r * k).sum(-1) / (r.norm(dim=-1) * k.norm(dim=-1))
        margin = min(margin, float(cosine.abs().min()))
    return margin


def read_folder(folder):
    """config.json and the tensors of a model folder."""
    import json
    from pathlib import Path

    import safetensors.torch

    config = json.loads((Path(folder) / "config.json").read_text())
    return config, safetensors.torch.load_file(str(Path(folder) / "model.safetensors"))
