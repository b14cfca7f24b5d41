"""EfficientAttention — drop-in for fairseq/modules/efficient_attention.py:11-60 (AttentionFunc,
attention, EfficientAttention): y = softmax(scale q k^T [causal mask, DropKey]) v per head.

As in the reference operator (fairseq/csrc/ops/attention_kernel.cu:39-131) the two products are
library GEMMs (cuBLAS through torch.matmul) around the attention-weight softmax, which is this
library's kernel (causal mask and DropKey built in, weights written once, in place of the
scores' dtype).  The (L x L) weights are materialised and saved for the backward like the
reference does; a single fused kernel over the chunk is not part of this build."""
import torch
import torch.nn as nn

from .. import ops


class AttentionFunction(torch.autograd.Function):
    """q, k: (B, L, N, H1); v: (B, L, N, H2); returns (B, L, N, H2)."""

    @staticmethod
    def forward(ctx, q, k, v, scale=1.0, dropout=0.0, use_causal_mask=True, training=True):
        ctx.qk_dtypes = (q.dtype, k.dtype)
        if q.dtype != v.dtype or k.dtype != v.dtype:
            # the Mega block's rotary embedding returns float32 queries and keys whatever the model's
            # dtype (relative_positional_bias.py:83-89): the products run in the values' dtype
            q, k = q.to(v.dtype), k.to(v.dtype)
        qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)       # (B, N, L, H)
        s = torch.matmul(qh, kh.transpose(-1, -2))                                # (B, N, L, L)
        if scale != 1.0:
            s = s * scale
        p = dropout if training else 0.0
        if p > 0.0:
            seed = int(torch.randint(0, 2 ** 62, (1,)).item())
            w = ops.attention_dropkey_softmax_fwd(s, p, use_causal_mask, seed, 0)
        else:
            w = ops.attention_softmax_fwd(s, use_causal_mask)
        y = torch.matmul(w, vh).transpose(1, 2)
        ctx.save_for_backward(q, k, v, w)
        ctx.scale, ctx.use_causal_mask = scale, use_causal_mask
        return y.contiguous()

    @staticmethod
    def backward(ctx, y_grad):
        q, k, v, w = ctx.saved_tensors
        qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        gh = y_grad.transpose(1, 2)                                               # (B, N, L, H2)
        v_grad = torch.matmul(w.transpose(-1, -2), gh)
        w_grad = torch.matmul(gh, vh.transpose(-1, -2))
        s_grad = ops.attention_softmax_bwd(w_grad, w, ctx.use_causal_mask)
        if ctx.scale != 1.0:
            s_grad = s_grad * ctx.scale
        q_grad = torch.matmul(s_grad, kh)
        k_grad = torch.matmul(s_grad.transpose(-1, -2), qh)
        return (q_grad.transpose(1, 2).contiguous().to(ctx.qk_dtypes[0]),
                k_grad.transpose(1, 2).contiguous().to(ctx.qk_dtypes[1]),
                v_grad.transpose(1, 2).contiguous(), None, None, None, None)


attention = AttentionFunction.apply


class EfficientAttention(nn.Module):
    def __init__(self, scale: float = 1.0, dropout: float = 0.0, use_causal_mask: bool = True) -> None:
        super().__init__()
        self._scale = scale
        self._dropout = dropout
        self._causal = use_causal_mask

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """q, k: (B, L, H1); v: (B, L, H2) -> (B, L, H2) (one head)."""
        out = attention(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), self._scale, self._dropout, self._causal,
                        self.training)
        return out.squeeze(2)

    def extra_repr(self) -> str:
        return 'causal={}, dropout={}'.format(self._causal, self._dropout)
