"""Linear attention with a fixed decay per head ("lightning attention").

For input ``h``: ``q = silu(W_q h)``, ``k = silu(W_k h)`` (heads x dim), ``v = silu(W_v h)``
(heads x vdim).  Per head a state matrix ``S`` [dim, vdim] runs through the request's tokens,
``S <- decay_h * S + k v^T`` and ``o = S^T q``; it starts at zero, is float32 and lives in the
request's state slot between steps.  The heads of ``o`` side by side are RMS-normalised together
(gain vector ``norm``), multiplied by ``sigmoid(W_g h)`` and projected by ``W_o``.

A step of single tokens runs the recurrence token by token; a step with prompt portions runs it in
chunks of 32 tokens (chunk sums, a walk over each request's chunks, outputs), which is the same
arithmetic in another order of additions, all float32.

q, k, v and the gate come from ONE matrix product with the four weights stacked; the activation of
q, k and v is applied in float32 inside the scan kernel, so that nothing that enters the recurrence
is rounded after the projection.  The mixer holds no pages: its cache is the state alone.
"""

from __future__ import annotations

from .base import Mixer, StateSpec, TensorSpec, register_part


class LightningAttention(Mixer):
    state_in_graphs = True   # the scan reads the step's numbers on the device and honours request_active

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int,
                 decay: tuple[float, ...], eps: float, names: dict[str, str] | None = None) -> None:
        if len(decay) != num_heads:
            raise ValueError("lightning attention needs one decay factor per head")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.key_dim = int(key_dim)
        self.value_dim = int(value_dim)
        self.decay = tuple(float(d) for d in decay)
        self.eps = float(eps)
        self.qk_width = self.num_heads * self.key_dim
        self.v_width = self.num_heads * self.value_dim
        self.names = dict(q="q", k="k", v="v", gate="g", out="o", norm="norm")
        self.names.update(names or {})

    @property
    def plan_key(self):
        return ("lightning",)

    def plan(self, host, cache):
        """Chunk work lists for a step with prompt portions (one list serves every lightning layer)."""
        return self.runtime.ops.plan_lightning(host)

    def state_spec(self) -> StateSpec:
        return StateSpec((self.num_heads, self.key_dim, self.value_dim), "float32")

    def tensor_specs(self) -> dict[str, TensorSpec]:
        n = self.names
        return {
            n["q"]: TensorSpec((self.qk_width, self.hidden_size)),
            n["k"]: TensorSpec((self.qk_width, self.hidden_size)),
            n["v"]: TensorSpec((self.v_width, self.hidden_size)),
            n["gate"]: TensorSpec((self.v_width, self.hidden_size)),
            n["out"]: TensorSpec((self.hidden_size, self.v_width)),
            n["norm"]: TensorSpec((self.v_width,), init="gain", role="vector"),
        }

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        n = self.names
        self.w_in = runtime.ops.prepare_weight(torch.cat([tensors[n[key]] for key in ("q", "k", "v", "gate")]))
        self.w_out = runtime.ops.prepare_weight(tensors[n["out"]])
        self.gain = tensors[n["norm"]].contiguous()
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float32, device=runtime.device)

    def forward(self, x, ctx, binding):
        import torch

        rt = self.runtime
        tokens = x.shape[0]
        width = 2 * self.qk_width + 2 * self.v_width
        proj = rt.workspace.get("lightning.proj", tokens, width, rt.dtype)
        rt.ops.linear(x, self.w_in, None, proj)
        mixed = rt.workspace.get("lightning.o", tokens, self.v_width, torch.float32)
        plan = getattr(ctx, "extras", {}).get(self.plan_key) or None
        limit = rt.ops.LIGHTNING_CHUNK_MAX_DIM
        if plan and self.key_dim <= limit and self.value_dim <= limit:
            # prompt portions: chunk sums, a short walk over the chunks, outputs, each wide
            rt.ops.lightning_chunked(proj, mixed, binding.state, self.decay_dev, ctx, plan, self.num_heads,
                                     self.key_dim, self.value_dim)
        else:
            rt.ops.lightning_scan(proj, mixed, binding.state, self.decay_dev, ctx, self.num_heads,
                                  self.key_dim, self.value_dim)
        gated = rt.workspace.get("lightning.gated", tokens, self.v_width, rt.dtype)
        rt.ops.lightning_gate_norm(mixed, proj[:, 2 * self.qk_width + self.v_width:], self.gain, self.eps, gated)
        update = rt.workspace.get("mixer.update32", tokens, self.hidden_size, torch.float32)
        return rt.ops.linear(gated, self.w_out, None, update)


register_part("mixer", "lightning", LightningAttention, replace=True)
