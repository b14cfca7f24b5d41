"""AttentionSoftmax — drop-in for fairseq/modules/attention_softmax.py:42-55: softmax of the
attention scores with the optional causal mask built in, forward and backward on the mega_b200
kernels.  DropKey (dropout > 0 while training) masks scores before the softmax with a
counter-based generator: the seed of a call is drawn from torch's default CPU generator, so
``torch.manual_seed`` makes a run repeatable; the masks equal the reference's in distribution,
not bit for bit (it reads curand's stream through its own thread layout)."""
import torch
import torch.nn as nn

from .. import ops


class AttentionSoftmaxFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, use_causal_mask, dropout=0.0):
        if dropout > 0.0:
            seed = int(torch.randint(0, 2 ** 62, (1,)).item())
            y = ops.attention_dropkey_softmax_fwd(x, dropout, use_causal_mask, seed, 0)
        else:
            y = ops.attention_softmax_fwd(x, use_causal_mask)
        ctx.save_for_backward(y)
        ctx.use_causal_mask = use_causal_mask
        return y

    @staticmethod
    def backward(ctx, y_grad):
        y, = ctx.saved_tensors  # dropped columns hold 0, so the plain softmax backward applies
        return ops.attention_softmax_bwd(y_grad, y, ctx.use_causal_mask), None, None


class AttentionSoftmax(nn.Module):
    def __init__(self, dropout: float = 0.0, use_causal_mask: bool = False) -> None:
        super().__init__()
        self._dropout = dropout
        self._causal = use_causal_mask

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return AttentionSoftmaxFunction.apply(x, self._causal, self._dropout if self.training else 0.0)

    def extra_repr(self) -> str:
        return 'causal={}, dropout={}'.format(self._causal, self._dropout)
