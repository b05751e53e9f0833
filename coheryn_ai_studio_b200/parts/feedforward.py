"""Dense gated feed-forward: y = W_down (act(W_gate x) * (W_up x)), no biases; act = silu (SwiGLU),
silu(g) = g / (1 + exp(-g)), or the tanh form of GELU, in float32
(crates/coheryn-engine/src/inference.rs:516-540, crates/coheryn-engine/src/cpu.rs:74-78).  ``swish_clamped`` with its
constant c is the variant g <- min(g, c), u <- clamp(u, -c, c), y = W_down (g sigmoid(1.702 g) (u + 1)).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.spec import TensorSpec
from .base import FeedForward, Runtime, StepContext, register_feed_forward


class GatedMLP(FeedForward):
    def __init__(self, runtime: Runtime, hidden_size: int, intermediate_size: int, activation: str,
                 tensors=("gate_proj.weight", "up_proj.weight", "down_proj.weight"), activation_constant=None,
                 float32_output: bool = False):
        """``tensors``: the local names of the gate, up and down matrices in the checkpoint.  ``activation_constant``:
        the constant of an activation that has one.  ``float32_output``: the down projection hands its result on in
        float32 (a block that normalises it before the residual add wants that)."""
        super().__init__(runtime)
        self.names = tuple(tensors)
        ops.gated_epilogue_word(activation, activation_constant)     # refuses an activation the epilogues lack
        self.activation, self.constant = activation, activation_constant
        self.out_dtype = torch.float32 if float32_output else None
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        H, I = self.hidden_size, self.intermediate_size
        g, u, d = self.names
        return {g: TensorSpec((I, H)), u: TensorSpec((I, H)), d: TensorSpec((H, I))}

    def bind(self, tensors):
        # One matrix product for gate and up, rows interleaved (2j = gate_j, 2j+1 = up_j) so
        # that the gated epilogue finds a pair in neighbouring output columns.
        g, u = tensors[self.names[0]], tensors[self.names[1]]
        self.w_gate_up = torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1]).contiguous()
        self.w_down = tensors[self.names[2]]

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        act = ops.gated_linear(x, self.w_gate_up, self.activation, param=self.constant)
        return ops.linear(act, self.w_down, out_dtype=self.out_dtype, partial_ok=self.partial_output)

    output_parts = 1

    # A block may take the output product over: it concatenates the activations of all its producers and multiplies them
    # by their stacked output matrices once (see ParallelResidual).
    def output_weights(self):
        return [self.w_down]

    def forward_open(self, x: torch.Tensor, step: StepContext, cache, outs) -> None:
        ops.gated_linear(x, self.w_gate_up, self.activation, out=outs[0], param=self.constant)

    def forward_into(self, x: torch.Tensor, step: StepContext, out: torch.Tensor) -> None:
        """The output written into ``out`` (float32 [1, T, H]): one of the summands that a block hands to the next norm."""
        ops.linear(ops.gated_linear(x, self.w_gate_up, self.activation, param=self.constant), self.w_down, out=out[0])


register_feed_forward("gated_mlp", GatedMLP)
