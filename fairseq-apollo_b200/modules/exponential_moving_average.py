"""MultiHeadEMA — drop-in for fairseq/modules/exponential_moving_average.py:13-94 on top of
BaseMovingLayer (fairseq/modules/base_moving_average.py:18-197), running on the mega_b200
CUDA kernels.

Same constructor, parameters (alpha, delta, beta (K, N, 1); gamma (K, N); omega (D)), state
dict keys, ``forward(x, padding_mask, incremental_state)`` with x of shape (B, D, L), the
``"ema_state"/{"prev_state"}`` incremental buffer, ``coeffs``/``kernel``/``step``/``one_step``,
``parameters_no_weight_decay`` and ``reorder_incremental_state``.

Where the reference class cannot run as written (omega (D,) multiplied into a (B, D, L)
tensor; ``_compute_kernel`` with a stale signature) this class implements what its working
sibling MultiHeadComplexEMA does: omega broadcast per channel and ``kernel`` returning
``(k, bias)``.  The state keeps the real-EMA convention h = sum p q^j x (p = sigmoid(alpha)*beta).
"""
import math
from collections import OrderedDict
from typing import Dict, Optional

import torch
from torch import Tensor, nn

from .. import ops
from ..functions import EMAFunction, needs_grad
from ..incremental_state import IncrementalStateMixin, require_no_grad


class MultiHeadEMA(IncrementalStateMixin, nn.Module):
    def __init__(self, embed_dim, ndim=2, bidirectional=False, truncation=None, shift=True):
        super().__init__()
        assert bidirectional or (truncation is None or truncation < 1), \
            'one directional moving average should not have positive trunction: {}'.format(truncation)
        self._parameters_no_weight_decay = OrderedDict()
        self.complex = False
        self.bidirectional = bidirectional
        self.truncation = truncation
        self.shift = shift
        self.embed_dim = embed_dim
        self.ndim = ndim
        self.scale = math.sqrt(1.0 / self.ndim)

        kernel_dim = 2 * embed_dim if self.bidirectional else embed_dim
        self.alpha = nn.Parameter(torch.empty(kernel_dim, ndim, 1))
        self.delta = nn.Parameter(torch.empty(kernel_dim, ndim, 1))
        self.beta = nn.Parameter(torch.empty(kernel_dim, ndim, 1))
        self.gamma = nn.Parameter(torch.empty(kernel_dim, ndim))
        self.omega = nn.Parameter(torch.empty(embed_dim))
        self._kernel = None
        self._coeffs = None

        self.register_parameters_no_weight_decay('alpha', self.alpha)
        self.register_parameters_no_weight_decay('delta', self.delta)
        self.reset_parameters()
        self.onnx_trace = False
        self.tpu = False

    # -- housekeeping identical in meaning to the reference ---------------------------
    def prepare_for_onnx_export_(self):
        self.onnx_trace = True

    def prepare_for_tpu_(self, **kwargs):
        self.tpu = True

    def register_parameters_no_weight_decay(self, name, param):
        self._parameters_no_weight_decay[name] = param

    def parameters_no_weight_decay(self):
        for name, param in self._parameters_no_weight_decay.items():
            yield name, param

    def reset_parameters(self):
        with torch.no_grad():
            nn.init.normal_(self.alpha, mean=0.0, std=0.2)
            nn.init.normal_(self.delta, mean=0.0, std=0.2)
            # beta alternates +1 / -1 along the ndim axis, plus small noise
            val = torch.ones(self.ndim, 1)
            val[1::2] = -1.0
            self.beta.normal_(mean=0.0, std=0.02).add_(val.to(self.beta))
            nn.init.normal_(self.gamma, mean=0.0, std=1.0)
            nn.init.normal_(self.omega, mean=0.0, std=1.0)

    def train(self, mode=True):
        self._coeffs = None  # cached coefficients are only valid while the parameters are frozen
        return super().train(mode)

    def _apply(self, fn, *args, **kwargs):
        self._coeffs = None
        return super()._apply(fn, *args, **kwargs)

    # -- coefficients / kernel -----------------------------------------------------------
    def _calc_coeffs(self):
        """(p, q, gamma_hat): p, q (K, N, 1), gamma_hat (K, N), all fp32 (CUDA kernel)."""
        self._coeffs = None
        p, q, g = ops.ema_coeffs(self.alpha, self.delta, self.beta, self.gamma)
        return p.unsqueeze(-1), q.unsqueeze(-1), g

    def coeffs(self):
        if self.training:
            return self._calc_coeffs()
        if self._coeffs is None:
            self._coeffs = self._calc_coeffs()
        return self._coeffs

    def _compute_kernel(self, length: int, hx: Optional[Tensor]):
        p, q, g = self.coeffs()
        k = ops.ema_kernel(p.squeeze(-1), q.squeeze(-1), g, length)
        b = None if hx is None else ops.ema_bias(q.squeeze(-1), g, hx, length)
        return k, b

    def kernel(self, length: int, hx: Optional[Tensor] = None):
        kernel_size = length if self.truncation is None or self.truncation < 1 else min(self.truncation, length)
        return self._compute_kernel(kernel_size, hx)

    # -- closed forms --------------------------------------------------------------------
    def one_step(self, x, hx=None):
        """x (B, D, 1) -> (out (B, D, 1) WITHOUT the omega residual, h (B, D, N))."""
        require_no_grad(x, self.alpha)
        p, q, g = self.coeffs()
        zero = torch.zeros_like(self.omega, dtype=torch.float32)
        y, h = ops.ema_step(x, p.squeeze(-1), q.squeeze(-1), g, zero, hx)
        return y, h

    def step(self, x, length, hx=None):
        """x (B, D, L) -> (out (B, D, L) WITHOUT the omega residual, h (B, D, N))."""
        require_no_grad(x, self.alpha)
        if length == 1:
            return self.one_step(x, hx=hx)
        p, q, g = self.coeffs()
        zero = torch.zeros_like(self.omega, dtype=torch.float32)
        return ops.ema_forward(x, p.squeeze(-1), q.squeeze(-1), g, zero, None, hx, want_state=True)

    # -- forward ---------------------------------------------------------------------------
    def forward(self, x, padding_mask: Optional[Tensor] = None,
                incremental_state: Optional[Dict[str, Dict[str, Optional[Tensor]]]] = None,
                activation: Optional[str] = None) -> Tensor:
        """x: (B, D, L) (any strides).  padding_mask: (B, L), non-zero = pad.
        ``activation='silu'`` fuses the caller's move_act into the epilogue."""
        bsz, embed_dim, seq_len = x.size()
        assert embed_dim == self.embed_dim
        assert activation in (None, 'silu')
        assert not self.bidirectional or incremental_state is None, \
            'Bidirectional EMA does not support incremental state'
        if needs_grad(x, self.alpha, self.delta, self.beta, self.gamma, self.omega):
            return self._forward_train(x, padding_mask, incremental_state, activation)
        p, q, g = self.coeffs()
        p, q = p.squeeze(-1), q.squeeze(-1)
        silu = activation == 'silu'
        if incremental_state is not None:
            saved_state = self._get_input_buffer(incremental_state)
            h = saved_state.get('prev_state')
            if seq_len == 1 and padding_mask is None:
                out, h = ops.ema_step(x, p, q, g, self.omega, h, silu=silu)
            else:
                out, h = ops.ema_forward(x, p, q, g, self.omega, padding_mask, h, want_state=True, silu=silu)
            saved_state['prev_state'] = h
            self._set_input_buffer(incremental_state, saved_state)
            return out
        return ops.ema_forward(x, p, q, g, self.omega, padding_mask, None, False,
                               bidirectional=self.bidirectional, shift=self.shift,
                               truncation=self.truncation, silu=silu)

    def _forward_train(self, x, padding_mask, incremental_state, activation):
        """Differentiable path: forward and backward kernels behind an autograd Function; the
        activation is applied by torch on the result, as the reference's caller does."""
        if incremental_state is not None:
            raise NotImplementedError("the incremental state is an inference feature: use torch.no_grad()")
        y = EMAFunction.apply(x, self.alpha, self.delta, self.beta, self.gamma, self.omega, padding_mask,
                              self.bidirectional, self.shift, self.truncation)
        return torch.nn.functional.silu(y) if activation == 'silu' else y

    def forward_time_major(self, x, padding_mask=None, incremental_state=None, activation=None):
        """x: (L, B, D) time-major; returns (L, B, D).  A strided view, no copy."""
        y = self.forward(x.permute(1, 2, 0), padding_mask, incremental_state, activation)
        return y.permute(2, 0, 1)

    # -- incremental state -------------------------------------------------------------------
    def _get_input_buffer(self, incremental_state):
        result = self.get_incremental_state(incremental_state, "ema_state")
        return result if result is not None else {}

    def _set_input_buffer(self, incremental_state, buffer):
        return self.set_incremental_state(incremental_state, "ema_state", buffer)

    def reorder_incremental_state(self, incremental_state, new_order: Tensor):
        return self._reorder_buffer(incremental_state, "ema_state", new_order)

    def extra_repr(self) -> str:
        return 'edim={}, ndim={}, bidirectional={}, trunction={}, shift={}'.format(
            self.embed_dim, self.ndim, self.bidirectional, self.truncation, self.shift)
