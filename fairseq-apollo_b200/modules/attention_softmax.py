"""AttentionSoftmax — drop-in for fairseq/modules/attention_softmax.py:42-55: softmax of the
attention scores with the optional causal mask built in, forward and backward on the mega_b200
kernels.  DropKey (dropout > 0 while training) is stochastic in the reference and is not built."""
import torch
import torch.nn as nn

from .. import ops


class AttentionSoftmaxFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, use_causal_mask):
        y = ops.attention_softmax_fwd(x, use_causal_mask)
        ctx.save_for_backward(y)
        ctx.use_causal_mask = use_causal_mask
        return y

    @staticmethod
    def backward(ctx, y_grad):
        y, = ctx.saved_tensors
        return ops.attention_softmax_bwd(y_grad, y, ctx.use_causal_mask), None


class AttentionSoftmax(nn.Module):
    def __init__(self, dropout: float = 0.0, use_causal_mask: bool = False) -> None:
        super().__init__()
        self._dropout = dropout
        self._causal = use_causal_mask

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.training and self._dropout > 0.0:
            raise NotImplementedError("DropKey (attention dropout inside the softmax) is not part of this build")
        return AttentionSoftmaxFunction.apply(x, self._causal)

    def extra_repr(self) -> str:
        return 'causal={}, dropout={}'.format(self._causal, self._dropout)
