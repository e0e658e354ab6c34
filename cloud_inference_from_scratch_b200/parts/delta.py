"""Generalized delta rule: a recurrent mixer whose state forgets per channel and unlearns along its key.

For input ``h``: ``r = W_r h``, ``k = W_k h``, ``v = W_v h`` (heads x dim each); a decay per head and key
channel ``w = exp(-exp(-1/2) * sigmoid(W_w2 tanh(W_w1 h) + w0))`` and a removal rate
``a = sigmoid(W_a h + a0)``.  With ``u = k / sqrt(sum(k^2) + 1e-6)`` per head, the state ``S`` [dim, dim]
of a head runs ``S <- diag(w) S - (a * u)(u^T S) + k v^T`` (both first terms from the old ``S``) and
``o = S^T r``.  Every head of ``o`` is divided by its own root mean square; the heads side by side are
multiplied by a gain vector and by ``sigmoid(W_g h)`` and projected by ``W_o``.

``S`` starts at zero, is float32 and lives in the request's state slot between steps.  r, k, v, the gate,
the removal projection and the first decay projection come from ONE matrix product with float32 results;
from there to the normalised output everything is float32 (only tanh(W_w1 h) is rounded to the compute
dtype, as the operand of the second decay product).  The mixer holds no pages.

The width of the low-rank decay projection is ``decay_rank``, or, if None, whatever the stored tensor has.

Tensor names (after the part's prefix): ``r``, ``k``, ``v``, ``g``, ``a``, ``a.b``, ``w1``, ``w2``, ``w0``,
``norm``, ``o``.
"""

from __future__ import annotations

from .base import Mixer, StateSpec, TensorSpec, register_part


class GeneralDelta(Mixer):
    state_in_graphs = True   # the scan reads the step's numbers on the device and honours request_active

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, eps: float,
                 decay_rank: int | None = None, names: dict[str, str] | None = None) -> None:
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.head_dim = int(head_dim)
        self.eps = float(eps)
        self.decay_rank = int(decay_rank) if decay_rank else -1     # -1: the file says
        self.width = self.num_heads * self.head_dim
        self.names = {key: key for key in ("r", "k", "v", "g", "a", "a.b", "w1", "w2", "w0", "norm", "o")}
        self.names.update(names or {})

    def state_spec(self) -> StateSpec:
        return StateSpec((self.num_heads, self.head_dim, self.head_dim), "float32")

    def tensor_specs(self) -> dict[str, TensorSpec]:
        n, width, hidden = self.names, self.width, self.hidden_size
        specs = {n[key]: TensorSpec((width, hidden)) for key in ("r", "k", "v", "g", "a")}
        specs[n["a.b"]] = TensorSpec((width,), role="vector")
        specs[n["w1"]] = TensorSpec((self.decay_rank, hidden))
        specs[n["w2"]] = TensorSpec((width, self.decay_rank))
        specs[n["w0"]] = TensorSpec((width,), role="vector")
        specs[n["norm"]] = TensorSpec((width,), init="gain", role="vector")
        specs[n["o"]] = TensorSpec((hidden, width))
        return specs

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        ops, n = runtime.ops, self.names
        largest = ops.require_delta()
        if self.head_dim > largest:
            raise ValueError(f"the delta-rule kernel takes heads of up to {largest}, got {self.head_dim}")
        self.rank = int(tensors[n["w1"]].shape[0])
        if tensors[n["w2"]].shape[1] != self.rank:
            raise ValueError("the two decay projections disagree about their inner width")
        self.w_in = ops.prepare_weight(torch.cat([tensors[n[key]] for key in ("r", "k", "v", "g", "a", "w1")]))
        self.w_decay = ops.prepare_weight(tensors[n["w2"]])
        self.w_out = ops.prepare_weight(tensors[n["o"]])
        self.decay_bias = tensors[n["w0"]].contiguous()
        self.removal_bias = tensors[n["a.b"]].contiguous()
        self.gain = tensors[n["norm"]].contiguous()

    def forward(self, x, ctx, binding):
        import torch

        rt = self.runtime
        ops = rt.ops
        tokens, width, f32 = x.shape[0], self.width, torch.float32
        proj = rt.workspace.get("delta.proj", tokens, 5 * width + self.rank, f32)
        ops.linear(x, self.w_in, None, proj)
        squashed = rt.workspace.get("delta.squashed", tokens, self.rank, rt.dtype)
        ops.tanh_rows(proj[:, 5 * width:], squashed)
        decay = rt.workspace.get("delta.decay", tokens, width, f32)
        ops.linear(squashed, self.w_decay, None, decay)
        mixed = rt.workspace.get("delta.o", tokens, width, f32)
        ops.delta_scan(proj, (0, width, 2 * width, 4 * width), decay, self.decay_bias, self.removal_bias, mixed,
                       binding.state, ctx, self.num_heads, self.head_dim)
        gated = rt.workspace.get("delta.gated", tokens, width, rt.dtype)
        ops.group_gate_norm(mixed, proj[:, 3 * width:4 * width], self.gain, self.eps, gated, self.num_heads)
        update = rt.workspace.get("mixer.update32", tokens, self.hidden_size, f32)
        return ops.linear(gated, self.w_out, None, update)


register_part("mixer", "general_delta", GeneralDelta, replace=True)
