"""MovingAverageGatedAttention — the Mega block that calls the EMA layer, on this library's kernels.

Drop-in for fairseq/modules/moving_average_gated_attention.py:26-470 (same constructor arguments,
parameter / buffer names and shapes, ``forward(x (B, L, D), padding_mask, incremental_state,
need_weights, attn_mask, before_attn_fn) -> (out, attn_weights)``, incremental-state keys
``"attn_state"/{"prev_key", "prev_value", "prev_key_padding_mask"}``).  What differs is which kernels
run the elementwise parts around the three projections (those stay library GEMMs, as in the
reference):

* ``x = norm(x); mx = move_act(move(x))``     one fused TimestepNorm -> EMA (+SiLU) launch that also
  returns the normalised activations for ``v_proj`` (``timestep_norm_ema``), or SequenceNorm -> EMA
  for the bidirectional block (``sequence_norm_ema``);
* ``silu(v_proj(x))``                          ``ops.gate_silu``;
* ``normalize(z) * (gamma + 1) + beta -> q, k`` ``ops.gate_qk`` (reads the z columns of the projection in place);
* ``attn * silu(r)``                           ``ops.gate_mul_silu``;
* ``residual + sigmoid(u) * (silu(hx + h_proj(.)) - residual)`` ``ops.gate_output``;
* causal chunked softmax attention             ``EfficientAttention`` (scores GEMM, this library's
  causal softmax, values GEMM) when ``efficient_attn`` is set, else the reference's explicit path.

Training (autograd enabled) takes the reference's own sequence of torch operations on top of the
differentiable modules; the fused elementwise kernels are inference paths.
"""
import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor, nn
from torch.nn import Parameter

from .. import ops
from ..functions import needs_grad
from ..incremental_state import IncrementalStateMixin
from .attention_softmax import AttentionSoftmax
from .complex_exponential_moving_average import MultiHeadComplexEMA
from .efficient_attention import EfficientAttention
from .exponential_moving_average import MultiHeadEMA
from .fused import sequence_norm_ema, timestep_norm_ema
from .sequence_norm import SequenceNorm
from .timestep_norm import TimestepNorm


class RotaryEmbedding(nn.Module):
    """Rotary position embedding of the query / key pair
    (fairseq/modules/relative_positional_bias.py:47-97): pairs of features are rotated by
    position * base^(-2j/dim); results are float32 like the reference's."""

    def __init__(self, embed_dim, max_positions, base=None):
        super().__init__()
        assert embed_dim % 2 == 0
        self.embed_dim, self.max_positions = embed_dim, max_positions
        self.base = 10000 if base is None else base
        inv = torch.tensor([self.base ** (j / embed_dim) for j in range(0, embed_dim, 2)], dtype=torch.float32)
        self.register_buffer("freqs", 1.0 / inv)
        self._table: Optional[Tensor] = None

    def _angles(self, start, end):
        if self._table is None or self._table.size(0) < end or self._table.device != self.freqs.device:
            n = max(end, self.max_positions)
            t = torch.arange(n, dtype=torch.float32, device=self.freqs.device)
            ang = torch.outer(t, self.freqs.float())
            self._table = torch.polar(torch.ones_like(ang), ang)
        return self._table[start:end]

    def rotary(self, x, start):
        rot = self._angles(start, start + x.size(1))
        xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
        return torch.view_as_real(xc * rot).flatten(2)

    def forward(self, xq, xk, qidx=0):
        return self.rotary(xq, qidx), self.rotary(xk, 0)

    def extra_repr(self):
        return 'dim={}, max positions={}, base={:.1f}'.format(self.embed_dim, self.max_positions, self.base)


class SimpleRelativePositionalBias(nn.Module):
    """Learned bias b[i - j] added to the scores (relative_positional_bias.py:13-44)."""

    def __init__(self, max_positions):
        super().__init__()
        self.max_positions = max_positions
        self.rel_pos_bias = Parameter(torch.empty(2 * max_positions - 1))
        nn.init.normal_(self.rel_pos_bias, mean=0, std=0.02)

    def forward(self, seq_len):
        if seq_len > self.max_positions:
            raise ValueError('Sequence length {} going beyond max length {}'.format(seq_len, self.max_positions))
        idx = torch.arange(seq_len, device=self.rel_pos_bias.device)
        rel = idx.view(1, -1) - idx.view(-1, 1) + (self.max_positions - 1)     # (key - query) offset
        return self.rel_pos_bias[rel]

    def extra_repr(self):
        return 'max positions={}'.format(self.max_positions)


class RMSNorm(nn.Module):
    """x / rms(x) * (weight + 1) over the last dimension (the reference's move_act='rmsnorm',
    norm_layer/layer_norm.py:40-58, is apex's fused RMS norm with the same offset-weight rule)."""

    def __init__(self, dim, eps=1e-5, elementwise_affine=True):
        super().__init__()
        self.eps = eps
        if elementwise_affine:
            self.weight = Parameter(torch.zeros(dim))
        else:
            self.register_parameter('weight', None)

    def forward(self, x):
        y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps)
        if self.weight is not None:
            y = y * (self.weight.float() + 1.0)
        return y.to(x.dtype)


class MovingAverageGatedAttention(IncrementalStateMixin, nn.Module):
    def __init__(self, embed_dim, zdim, hdim, ndim, dropout=0.0, attention_dropout=0.0, hidden_dropout=0.0,
                 efficient_attn=False, attention_activation='softmax', bidirectional=False, chunk_size=-1,
                 moving_layer='ema', moving_act='rmsnorm', truncation=None, norm_num_groups=None, norm_affine=True,
                 norm_eps=1e-5, rel_pos_bias='simple', max_positions=1024, init_mode='bert'):
        super().__init__()
        self.embed_dim, self.hdim, self.zdim, self.ndim = embed_dim, hdim, zdim, ndim
        self.attention_activation = attention_activation
        self.init_mode = init_mode
        self.dropout_p, self.hidden_dropout_p, self.attention_dropout_p = dropout, hidden_dropout, attention_dropout
        self.chunk_size, self.bidirectional = chunk_size, bidirectional
        self.efficient_attn = self.attn_softmax = None
        if efficient_attn:
            assert attention_activation == 'softmax'
            if bidirectional:
                self.attn_softmax = AttentionSoftmax(dropout=attention_dropout, use_causal_mask=False)
            else:
                self.efficient_attn = EfficientAttention(dropout=attention_dropout, use_causal_mask=True, scale=1.0)
        if bidirectional:
            self.norm = SequenceNorm(embed_dim, num_groups=norm_num_groups, eps=norm_eps)
        else:
            # (the reference leaves prior_count at 0, which only the grouped form accepts; a per-feature
            # TimestepNorm needs at least two pseudo-samples, norm_layer/timestep_norm.py:79-83)
            self.norm = TimestepNorm(embed_dim, num_groups=norm_num_groups, eps=norm_eps,
                                     prior_count=0 if norm_num_groups not in (None, embed_dim) else 2)
        if moving_layer == 'ema':
            self.move = MultiHeadEMA(embed_dim, ndim=ndim, bidirectional=bidirectional, truncation=truncation)
        elif moving_layer == 'cema':
            self.move = MultiHeadComplexEMA(embed_dim, ndim=ndim, bidirectional=bidirectional, truncation=truncation)
        else:
            raise ValueError("Unknown moving type: {}".format(moving_layer))
        assert moving_act in ('rmsnorm', 'silu')
        self.move_act = RMSNorm(embed_dim, eps=norm_eps, elementwise_affine=norm_affine) if moving_act == 'rmsnorm' \
            else nn.SiLU()
        self.v_proj = nn.Linear(embed_dim, hdim, bias=True)
        self.mx_proj = nn.Linear(embed_dim, zdim + hdim + 2 * embed_dim, bias=True)
        self.h_proj = nn.Linear(hdim, embed_dim, bias=False)
        self.gamma = Parameter(torch.zeros(2, zdim))
        self.beta = Parameter(torch.zeros(2, zdim))
        self.max_positions = max_positions
        span = max_positions if chunk_size < 0 else chunk_size
        if rel_pos_bias == 'simple':
            self.rel_pos_bias = SimpleRelativePositionalBias(span)
        elif rel_pos_bias == 'rotary':
            self.rel_pos_bias = RotaryEmbedding(zdim, span)
        else:
            raise ValueError('unknown relative position bias: {}'.format(rel_pos_bias))
        assert init_mode in ('bert', 'xavier', 'he')
        self.reset_parameters(init_mode)

    def reset_parameters(self, mode):
        for lin in (self.v_proj, self.mx_proj, self.h_proj):
            if mode == 'bert':
                nn.init.normal_(lin.weight, mean=0.0, std=0.02)
            elif mode == 'he':
                nn.init.kaiming_normal_(lin.weight, a=math.sqrt(5.0))
            else:
                nn.init.xavier_uniform_(lin.weight)
        nn.init.constant_(self.v_proj.bias, 0.0)
        nn.init.constant_(self.mx_proj.bias, 0.0)
        nn.init.constant_(self.gamma, 0.0)
        nn.init.constant_(self.beta, 0.0)

    # ------------------------------------------------------------------ attention weights
    def _scores(self, q, k):
        """Rotary positions or the learned relative bias applied, raw scores (B*K, Cq, Ck)."""
        slen = k.size(1)
        if isinstance(self.rel_pos_bias, RotaryEmbedding):
            qidx = slen - 1 if slen != q.size(1) else 0
            q, k = self.rel_pos_bias(q, k, qidx=qidx)
            return torch.bmm(q, k.transpose(1, 2)), None
        bias = self.rel_pos_bias(slen)
        if slen != q.size(1):
            assert q.size(1) == 1
            bias = bias[-1:]
        return torch.bmm(q, k.transpose(1, 2)), bias

    def softmax_attention(self, q, k, padding_mask, attn_mask, before_attn_fn):
        qk, bias = self._scores(q, k)
        if bias is not None:
            qk = qk + bias
        if attn_mask is not None:
            assert self.attn_softmax is None
            qk = qk + attn_mask
        if padding_mask is not None:
            all_pad = padding_mask.all(dim=-1, keepdim=True)
            padding_mask = torch.logical_and(padding_mask, ~all_pad)
            qk = qk.masked_fill(padding_mask.unsqueeze(1).to(torch.bool), float('-inf'))
        if before_attn_fn:
            return qk
        if self.attn_softmax is not None:
            return self.attn_softmax(qk)
        w = F.softmax(qk.float(), dim=-1).to(qk)
        return F.dropout(w, self.attention_dropout_p, self.training)

    def element_attention(self, q, k, padding_mask, attn_mask, before_attn_fn):
        slen = k.size(1)
        if padding_mask is not None:
            lengths = slen - padding_mask.sum(dim=-1, keepdim=True)
            len_scale = torch.rsqrt(lengths.clamp(min=1.0)).to(q).unsqueeze(-1)
            keep = 1.0 - padding_mask.to(q)
        else:
            len_scale, keep = 1.0 / math.sqrt(slen), None
        if attn_mask is not None:
            len_scale = torch.rsqrt(attn_mask.float().sum(dim=-1, keepdim=True)).to(q)
        qk, bias = self._scores(q, k)
        qk = qk * len_scale
        if bias is not None:
            qk = qk + bias
        if before_attn_fn:
            return qk
        if self.attention_activation == 'relu2':
            w = torch.square(F.relu(qk)).to(qk)
        elif self.attention_activation == 'laplace':
            mu, sigma = math.sqrt(0.5), math.sqrt(0.25 / math.pi)
            w = (0.5 * (1.0 + torch.erf((qk.float() - mu) / (sigma * math.sqrt(2.0))))).to(qk)
        else:
            raise ValueError('Unknown attention activation function: {}'.format(self.attention_activation))
        if keep is not None:
            w = w * keep.unsqueeze(1)
        if attn_mask is not None:
            w = w * attn_mask
        return F.dropout(w, self.attention_dropout_p, self.training)

    # ------------------------------------------------------------------ forward
    def forward(self, x, padding_mask: Optional[Tensor] = None,
                incremental_state: Optional[Dict[str, Dict[str, Optional[Tensor]]]] = None,
                need_weights: bool = False, attn_mask: Optional[Tensor] = None,
                before_attn_fn: bool = False) -> Tuple[Tensor, Optional[Tensor]]:
        """x: (B, L, D) -> (out (B, L, D), attention weights or None)."""
        bsz, seq_len, embed_dim = x.size()
        assert embed_dim == self.embed_dim
        saved_state = self._get_input_buffer(incremental_state) if incremental_state is not None else None
        residual = x
        train = needs_grad(x, *self.parameters())
        silu_act = isinstance(self.move_act, nn.SiLU)
        fused_elementwise = not train and x.is_cuda

        # ---- norm -> EMA (-> SiLU): mx (B, L, D) and the normalised activations xn (B, L, D)
        if self.bidirectional:
            xn_t = self.norm(x.transpose(1, 2), padding_mask)
            xn = xn_t.transpose(1, 2)
            mx = self.move(xn_t, padding_mask, None, 'silu' if (silu_act and not train) else None).transpose(1, 2)
            if silu_act and train:
                mx = F.silu(mx)
        elif train:
            xn = self.norm(x, padding_mask=padding_mask, incremental_state=incremental_state)
            mx = self.move(xn.transpose(1, 2), padding_mask, incremental_state).transpose(1, 2)
            if silu_act:
                mx = F.silu(mx)
        else:
            mx, xn = timestep_norm_ema(self.norm, self.move, x, padding_mask, incremental_state,
                                       activation='silu' if silu_act else None, return_normed=True)
        if not silu_act:
            mx = self.move_act(mx)
        mx = F.dropout(mx, self.hidden_dropout_p, self.training)

        # ---- projections and gates
        v_lin = self.v_proj(xn)
        base = self.mx_proj(mx)
        D, S, E = self.embed_dim, self.zdim, self.hdim
        u, z, r, hx = base[..., :D], base[..., D:D + S], base[..., D + S:D + S + E], base[..., D + S + E:]
        # rotary positions in the same kernel as the query / key affine: the plain (non-incremental) call of the
        # efficient-attention branch, where row (b, t) sits at position t % period of its chunk
        period = self.chunk_size if 1 < self.chunk_size < seq_len else seq_len
        fused_rotary = (fused_elementwise and self.efficient_attn is not None and saved_state is None
                        and isinstance(self.rel_pos_bias, RotaryEmbedding) and seq_len % period == 0
                        and period <= self.rel_pos_bias.max_positions)
        if fused_elementwise:
            v = ops.gate_silu(v_lin)
            if fused_rotary:
                q, k = ops.gate_qk_rotary(z, self.gamma, self.beta, self.rel_pos_bias._angles(0, period), period)
            else:
                q, k = ops.gate_qk(z, self.gamma, self.beta, eps=1e-5)
        else:
            v = F.silu(v_lin)
            zn = F.normalize(z, p=2, dim=-1, eps=1e-5)
            zq = zn.unsqueeze(2) * (self.gamma + 1.0) + self.beta
            q, k = torch.unbind(zq, dim=2)

        # ---- incremental keys / values (moving_average_gated_attention.py:332-371)
        if saved_state is not None:
            if "prev_key" in saved_state:
                k = torch.cat([saved_state["prev_key"], k], dim=1)
            if "prev_value" in saved_state:
                v = torch.cat([saved_state["prev_value"], v], dim=1)
            padding_mask = self._append_prev_padding_mask(padding_mask, saved_state.get("prev_padding_mask"),
                                                          bsz, k.size(1))
            keep_kv = self.chunk_size < 0 or (k.size(1) % self.chunk_size) != 0
            if keep_kv:
                saved_state["prev_key"], saved_state["prev_value"] = k, v
                saved_state["prev_key_padding_mask"] = padding_mask
            else:
                for key in ("prev_key", "prev_value", "prev_key_padding_mask"):
                    saved_state.pop(key, None)
            self._set_input_buffer(incremental_state, saved_state)

        # ---- chunking: (B, L, .) -> (B*K, C, .)
        if 1 < self.chunk_size < seq_len:
            q = q.reshape(bsz * (seq_len // self.chunk_size), self.chunk_size, S)
        ctx_len = k.size(1)
        if 1 < self.chunk_size < ctx_len:
            nc = ctx_len // self.chunk_size
            k = k.reshape(bsz * nc, self.chunk_size, S)
            v = v.reshape(bsz * nc, self.chunk_size, E)
            if padding_mask is not None:
                padding_mask = padding_mask.reshape(bsz * nc, self.chunk_size)
        if padding_mask is not None and padding_mask.dim() == 0:
            padding_mask = None

        # ---- attention
        attn_weights = None
        if self.efficient_attn is not None:
            assert isinstance(self.rel_pos_bias, RotaryEmbedding)
            if fused_rotary:
                qr, kr = q, k
            else:
                qidx = k.size(1) - 1 if k.size(1) != q.size(1) else 0
                qr, kr = self.rel_pos_bias(q, k, qidx=qidx)
            attn = self.efficient_attn(qr.to(v.dtype), kr.to(v.dtype), v).view(bsz, seq_len, E)
        else:
            if self.attention_activation == 'softmax':
                attn_weights = self.softmax_attention(q, k, padding_mask, attn_mask, before_attn_fn)
            else:
                attn_weights = self.element_attention(q, k, padding_mask, attn_mask, before_attn_fn)
            if before_attn_fn:
                return attn_weights, v
            attn = torch.bmm(attn_weights.to(v.dtype), v).view(bsz, seq_len, E)

        # ---- output gate
        if fused_elementwise and self.hidden_dropout_p == 0.0 and self.dropout_p == 0.0:
            gated = ops.gate_mul_silu(attn, r)
            out = ops.gate_output(residual, u, hx, self.h_proj(gated))
        else:
            gated = F.dropout(attn * F.silu(r), self.hidden_dropout_p, self.training)
            h = F.dropout(F.silu(hx + self.h_proj(gated)), self.dropout_p, self.training)
            out = torch.addcmul(residual, torch.sigmoid(u), h - residual)
        return (out, attn_weights) if need_weights else (out, None)

    # ------------------------------------------------------------------ incremental state
    def _get_input_buffer(self, incremental_state):
        result = self.get_incremental_state(incremental_state, "attn_state")
        return result if result is not None else {}

    def _set_input_buffer(self, incremental_state, buffer):
        return self.set_incremental_state(incremental_state, "attn_state", buffer)

    def reorder_incremental_state(self, incremental_state, new_order: Tensor):
        return self._reorder_buffer(incremental_state, "attn_state", new_order)

    @staticmethod
    def _append_prev_padding_mask(padding_mask, prev_padding_mask, batch_size, seq_len):
        if prev_padding_mask is not None and padding_mask is not None:
            return torch.cat([prev_padding_mask, padding_mask], dim=1)
        if prev_padding_mask is not None:
            filler = torch.zeros((batch_size, seq_len - prev_padding_mask.size(1)), device=prev_padding_mask.device)
            return torch.cat([prev_padding_mask, filler.bool()], dim=1)
        if padding_mask is not None:
            filler = torch.zeros((batch_size, seq_len - padding_mask.size(1)), device=padding_mask.device)
            return torch.cat([filler.bool(), padding_mask], dim=1)
        return None

    def extra_repr(self) -> str:
        return 'edim={}, zdim={}, hdim={}, ndim={}, chunk={}, attn_act={}, bidir={}, init={}'.format(
            self.embed_dim, self.zdim, self.hdim, self.ndim, self.chunk_size, self.attention_activation,
            self.bidirectional, self.init_mode)
