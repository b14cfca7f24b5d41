"""MultiHeadComplexEMA — drop-in for fairseq/modules/complex_exponential_moving_average.py:15-113
on top of BaseMovingLayer (fairseq/modules/base_moving_average.py:18-197), on the mega_b200 CUDA
kernels.

Same constructor, parameters (alpha, delta (K, N, 1); theta (K, 1, 1); gamma (K, N, 2); omega
(D, 1)), state-dict keys, ``forward(x (B, D, L), padding_mask, incremental_state)``, the
``"ema_state"/{"prev_state"}`` buffer holding a complex64 (B, D, N) state, ``coeffs``, ``kernel``,
``step``, ``one_step``, ``parameters_no_weight_decay`` and ``reorder_incremental_state``.
With autograd enabled the layer runs through an autograd Function whose forward and backward are
library kernels (no incremental state on that path).
"""
import math
from collections import OrderedDict
from typing import Dict, Optional

import torch
from torch import Tensor, nn

from .. import ops
from ..functions import ComplexEMAFunction, needs_grad
from ..incremental_state import IncrementalStateMixin, require_no_grad


class MultiHeadComplexEMA(IncrementalStateMixin, nn.Module):
    def __init__(self, embed_dim, ndim=2, bidirectional=False, truncation=None, shift=True):
        super().__init__()
        assert bidirectional or (truncation is None or truncation < 1), \
            'one directional moving average should not have positive trunction: {}'.format(truncation)
        self._parameters_no_weight_decay = OrderedDict()
        self.complex = True
        self.bidirectional = bidirectional
        self.truncation = truncation
        self.shift = shift
        self.embed_dim = embed_dim
        self.ndim = ndim
        self.scale = math.sqrt(1.0 / self.ndim)

        kernel_dim = 2 * embed_dim if self.bidirectional else embed_dim
        self.alpha = nn.Parameter(torch.empty(kernel_dim, ndim, 1))
        self.delta = nn.Parameter(torch.empty(kernel_dim, ndim, 1))
        self.theta = nn.Parameter(torch.empty(kernel_dim, 1, 1))
        self.gamma = nn.Parameter(torch.empty(kernel_dim, ndim, 2))
        self.omega = nn.Parameter(torch.empty(embed_dim, 1))
        self._coeffs = None

        self.register_parameters_no_weight_decay('alpha', self.alpha)
        self.register_parameters_no_weight_decay('delta', self.delta)
        self.register_parameters_no_weight_decay('theta', self.theta)
        self.reset_parameters()
        self.onnx_trace = False
        self.tpu = False

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
            # theta: log-spaced base frequencies in (0, 1), shuffled over the channels, stored as logits
            step = math.log(self.embed_dim) / self.embed_dim
            freqs = torch.exp(torch.arange(1, self.embed_dim + 1) * -step)
            freqs = freqs[torch.randperm(self.embed_dim)].to(self.theta).view(self.embed_dim, 1, 1)
            if self.bidirectional:
                freqs = freqs.repeat(2, 1, 1)
            self.theta.copy_(torch.log(freqs / (1.0 - freqs)))
            nn.init.normal_(self.gamma, mean=0.0, std=1.0)
            self.gamma[:, :, 1] = 0.
            nn.init.normal_(self.omega, mean=0.0, std=1.0)

    def train(self, mode=True):
        self._coeffs = None
        return super().train(mode)

    def _apply(self, fn, *args, **kwargs):
        self._coeffs = None
        return super()._apply(fn, *args, **kwargs)

    # -- coefficients / kernel -----------------------------------------------------------
    def _calc_coeffs(self):
        """p (K, N, 1) fp32, q (K, N, 1) complex64, gamma_hat (K, N) complex64."""
        self._coeffs = None
        p, q, g = ops.cema_coeffs(self.alpha, self.delta, self.theta, self.gamma)
        return p.unsqueeze(-1), q.unsqueeze(-1), g

    def coeffs(self):
        if self.training:
            return self._calc_coeffs()
        if self._coeffs is None:
            self._coeffs = self._calc_coeffs()
        return self._coeffs

    def _compute_kernel(self, length: int, hx: Optional[Tensor]):
        """(k (K, length) fp32, bias (B, D, length) fp32 of a carried state or None)."""
        p, q, g = self.coeffs()
        k = ops.cema_kernel(p.squeeze(-1), q.squeeze(-1), g, length)
        b = None
        if hx is not None:
            # output of the carried state alone: the layer run on a zero input from that state
            zero_x = torch.zeros(hx.shape[0], self.embed_dim, length, device=hx.device, dtype=torch.float32)
            zero_w = torch.zeros(self.embed_dim, device=hx.device, dtype=torch.float32)
            b = ops.cema_forward(zero_x, p.squeeze(-1), q.squeeze(-1), g, zero_w, None, hx)
        return k, b

    def kernel(self, length: int, hx: Optional[Tensor] = None):
        kernel_size = length if self.truncation is None or self.truncation < 1 else min(self.truncation, length)
        return self._compute_kernel(kernel_size, hx)

    # -- closed forms --------------------------------------------------------------------
    def one_step(self, x, hx=None):
        """x (B, D, 1) -> (out (B, D, 1) WITHOUT the omega residual, h (B, D, N) complex64)."""
        require_no_grad(x, self.alpha)
        p, q, g = self.coeffs()
        zero = torch.zeros(self.embed_dim, device=x.device, dtype=torch.float32)
        return ops.cema_step(x, p.squeeze(-1), q.squeeze(-1), g, zero, hx)

    def step(self, x, length, hx=None):
        """x (B, D, L) -> (out (B, D, L) WITHOUT the omega residual, h (B, D, N) complex64)."""
        require_no_grad(x, self.alpha)
        if length == 1:
            return self.one_step(x, hx=hx)
        p, q, g = self.coeffs()
        zero = torch.zeros(self.embed_dim, device=x.device, dtype=torch.float32)
        return ops.cema_forward(x, p.squeeze(-1), q.squeeze(-1), g, zero, None, hx, want_state=True)

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
        if needs_grad(x, self.alpha, self.delta, self.theta, self.gamma, self.omega):
            # differentiable path: forward and backward kernels behind an autograd Function; the
            # activation is applied by torch on the result, as the reference's caller does
            if incremental_state is not None:
                raise NotImplementedError("the incremental state is an inference feature: use torch.no_grad()")
            y = ComplexEMAFunction.apply(x, self.alpha, self.delta, self.theta, self.gamma, self.omega,
                                         padding_mask, self.bidirectional, self.shift, self.truncation)
            return torch.nn.functional.silu(y) if activation == 'silu' else y
        p, q, g = self.coeffs()
        p, q = p.squeeze(-1), q.squeeze(-1)
        silu = activation == 'silu'
        if incremental_state is not None:
            saved_state = self._get_input_buffer(incremental_state)
            h = saved_state.get('prev_state')
            if seq_len == 1 and padding_mask is None:
                out, h = ops.cema_step(x, p, q, g, self.omega, h, silu=silu)
            else:
                out, h = ops.cema_forward(x, p, q, g, self.omega, padding_mask, h, want_state=True, silu=silu)
            saved_state['prev_state'] = h
            self._set_input_buffer(incremental_state, saved_state)
            return out
        return ops.cema_forward(x, p, q, g, self.omega, padding_mask, None, False,
                                bidirectional=self.bidirectional, shift=self.shift,
                                truncation=self.truncation, silu=silu)

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
