"""Hyper-connections: a sublayer reads a weighted sum of several residual streams and writes
every stream back as a mix of the old streams plus its own result.

For one sublayer with result ``y`` and tensors ``in`` [S], ``out`` [S], ``mix`` [S, S] (indexed
[from, to]):  ``u = sum_s in[s] * x_s`` is what the sublayer's norm reads, and afterwards, all
streams at once from the old ones, ``x_t <- sum_s mix[s, t] * x_s + out[t] * y``.  The write is not
done here: it travels as a ``StreamUpdate`` to whoever reads the streams next, whose kernel applies
it in float32 together with its own read and norm.
"""

from __future__ import annotations

from ..lazy import StreamUpdate
from .base import Connection, TensorSpec, register_part


class HyperConnection(Connection):
    def __init__(self, streams: int) -> None:
        if streams < 1:
            raise ValueError("a hyper-connection needs at least one stream")
        self.streams = int(streams)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        s = self.streams
        return {
            "in": TensorSpec((s,), init="gain", role="vector"),
            "out": TensorSpec((s,), init="gain", role="vector"),
            "mix": TensorSpec((s, s), init="eye", role="vector"),
        }

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        self.w_in = tensors["in"].contiguous()
        self.w_out = tensors["out"].contiguous()
        self.w_mix = tensors["mix"].contiguous()

    def read_weights(self):
        return self.w_in

    def pending(self, y):
        return StreamUpdate(y, self.w_mix, self.w_out)


register_part("connection", "hyper", HyperConnection, replace=True)
