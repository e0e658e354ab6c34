"""Plain, slow implementation of the Zisesun decoder: one function per mechanism, float64 on
the CPU, token by token where the design is recurrent.  It shares no code with the engine; the
GPU tests hold the engine to it.

Notation: ``h`` is a sublayer's input [T, width]; a weight ``W`` is stored [out, in] and applied
as ``h @ W.T``; ``p`` maps a layer's tensor names (without the layer prefix) to float64 tensors.
"""

from __future__ import annotations

import torch

F = torch.float64


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def single_gain_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose gain is one number for all coordinates."""
    return rms_divide(x, eps) * gain.reshape(())


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def embedding(tokens: list[int], table: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Token row plus the learned vector of the token's position (positions count from 0)."""
    ids = torch.tensor(tokens, dtype=torch.long)
    return table[ids] + positions[: len(tokens)]


def lightning_recurrence(q, k, v, decay, state=None):
    """q, k [T, heads, dim], v [T, heads, vdim] (after their activation); per head the state S
    [dim, vdim] runs S <- decay * S + k v^T and o = S^T q.  Returns o [T, heads, vdim] and the
    states after the last token [heads, dim, vdim]."""
    tokens, heads, dim = q.shape
    vdim = v.shape[-1]
    out = torch.zeros(tokens, heads, vdim, dtype=F)
    state = torch.zeros(heads, dim, vdim, dtype=F) if state is None else state.clone().to(F)
    for head in range(heads):
        for t in range(tokens):
            state[head] = float(decay[head]) * state[head] + torch.outer(k[t, head], v[t, head])
            out[t, head] = state[head].T @ q[t, head]
    return out, state


def lightning_mixer(h: torch.Tensor, p: dict, mixer: dict, eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head; heads normalised together, gated, projected."""
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    tokens = h.shape[0]
    q = silu(h @ p["mix.q"].T).view(tokens, heads, dim)
    k = silu(h @ p["mix.k"].T).view(tokens, heads, dim)
    v = silu(h @ p["mix.v"].T).view(tokens, heads, vdim)
    out, _ = lightning_recurrence(q, k, v, mixer["decay"])
    flat = out.reshape(tokens, heads * vdim)
    flat = rms_divide(flat, eps) * p["mix.norm"]
    flat = flat * torch.sigmoid(h @ p["mix.g"].T)
    return flat @ p["mix.o"].T


def windowed_softmax_attention(q, k, v, scale, window, r1, r2, first_position=0):
    """q [T, heads, dim] at positions first_position.., k [N, groups, dim], v [N, groups, vdim] at
    positions 0..N-1 (N = first_position + T).  Query head h reads group h // (heads / groups); query
    position i sees keys j with 0 <= i - j < window (window 0: every j <= i); the score is
    q.k * scale - r1_h * ln(1 + r2_h * (i - j)) (r1 None: no penalty); ordinary softmax."""
    tokens, heads, _ = q.shape
    groups = k.shape[1]
    out = torch.zeros(tokens, heads, v.shape[-1], dtype=F)
    for head in range(heads):
        group = head // (heads // groups)
        for t in range(tokens):
            i = first_position + t
            first = max(0, i - window + 1) if window else 0
            keys = torch.arange(first, i + 1)
            score = (k[keys, group] @ q[t, head]) * scale
            if r1 is not None:
                score = score - float(r1[head]) * torch.log1p(float(r2[head]) * (i - keys).to(F))
            out[t, head] = torch.softmax(score, 0) @ v[keys, group]
    return out


def window_attention_mixer(h: torch.Tensor, p: dict, mixer: dict, eps: float) -> torch.Tensor:
    """Grouped-query softmax attention without rotation: q and k normalised over their whole
    projection, every value head divided by its own root mean square, a logarithmic distance
    penalty per head, and a window of ``mask.size`` keys (all earlier keys when there is no mask)."""
    heads, groups, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    tokens = h.shape[0]
    q = h @ p["mix.q"].T + p["mix.q.b"]
    k = h @ p["mix.k"].T + p["mix.k.b"]
    v = h @ p["mix.v"].T + p["mix.v.b"]
    q = (rms_divide(q, eps) * p["mix.q.norm"]).view(tokens, heads, dim)
    k = (rms_divide(k, eps) * p["mix.k.norm"]).view(tokens, groups, dim)
    v = rms_divide(v.view(tokens, groups, vdim), eps)
    window = (mixer.get("mask") or {}).get("size", 0)
    out = windowed_softmax_attention(q, k, v, mixer["scale"], window, p["mix.r1"], p["mix.r2"])
    return out.reshape(tokens, heads * vdim) @ p["mix.o"].T


def routed_experts(h: torch.Tensor, p: dict, mlp: dict) -> torch.Tensor:
    """Softmax router over all experts; the choice adds a correction to the scores, the mixing
    weights are the uncorrected scores of the chosen experts, not renormalised."""
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.softmax(h @ p["mlp.router"].T, -1)
    chosen = torch.topk(scores + p["mlp.correction"], top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            inner = silu(h[t] @ p[f"mlp.e{e}.gate"].T) * (h[t] @ p[f"mlp.e{e}.up"].T)
            out[t] += scores[t, e] * (inner @ p[f"mlp.e{e}.down"].T)
    assert experts == scores.shape[-1]
    return out


def run_mixer(kind: str, h, p, mixer, eps):
    if kind == "lightning":
        return lightning_mixer(h, p, mixer, eps)
    if kind == "attention":
        return window_attention_mixer(h, p, mixer, eps)
    raise ValueError(kind)


def hyper_sublayer(streams: torch.Tensor, p: dict, which: str, gain: torch.Tensor, eps: float, fn):
    """streams [S, T, width].  Reads u = sum_s in[s] x_s, runs y = fn(norm(u)), and writes every
    stream from the old ones: x_t <- sum_s mix[s, t] x_s + out[t] y."""
    u = torch.einsum("s,std->td", p[which + ".in"], streams)
    y = fn(single_gain_norm(u, gain, eps))
    return torch.einsum("sr,std->rtd", p[which + ".mix"], streams) + p[which + ".out"][:, None, None] * y


def layer_tensors(tensors: dict, index: int) -> dict:
    prefix = f"l{index}."
    return {name[len(prefix):]: value.to(F) for name, value in tensors.items() if name.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens: list[int], keep_layers: bool = False):
    """Logits [T, vocab] of one request fed whole (float64); with ``keep_layers`` also the sum of
    the streams after every layer run."""
    eps = float(config["norm"]["eps"])
    streams_count = config.get("streams")
    x = embedding(tokens, tensors["embed"].to(F), tensors["pos"].to(F))
    streams = x.unsqueeze(0).repeat(streams_count or 1, 1, 1)
    kept = []
    for index, layer in enumerate(config["layers"]):
        owner = index
        while config["layers"][owner].get("weights_of") is not None:     # tensors of an earlier layer
            owner = config["layers"][owner]["weights_of"]
        p = layer_tensors(tensors, owner)
        mixer_fn = lambda h, layer=layer, p=p: run_mixer(layer["type"], h, p, layer["mixer"], eps)  # noqa: E731
        ff_fn = lambda h, layer=layer, p=p: routed_experts(h, p, layer["mlp"])  # noqa: E731
        if streams_count:
            streams = hyper_sublayer(streams, p, "hc1", p["norm1"], eps, mixer_fn)
            if layer.get("mlp"):
                streams = hyper_sublayer(streams, p, "hc2", p["norm2"], eps, ff_fn)
        else:
            streams = streams + mixer_fn(single_gain_norm(streams[0], p["norm1"], eps))
            if layer.get("mlp"):
                streams = streams + ff_fn(single_gain_norm(streams[0], p["norm2"], eps))
        kept.append(streams.sum(0))
    x = single_gain_norm(streams.sum(0), tensors["final.norm"].to(F), eps)
    logits = x @ tensors["head"].to(F).T
    return (logits, torch.stack(kept)) if keep_layers else logits


def read_folder(folder):
    """config.json and the tensors of a model folder."""
    import json
    from pathlib import Path

    import safetensors.torch

    config = json.loads((Path(folder) / "config.json").read_text())
    return config, safetensors.torch.load_file(str(Path(folder) / "model.safetensors"))


def greedy(config: dict, tensors: dict, prompt: list[int], count: int) -> list[int]:
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(forward(config, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt):]
