"""Linear attention: a recurrence over a state of fixed size per request instead of keys and values
of every token."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Part, StateNeed, register_mixer


@register_mixer("decay_linear_attention")
class DecayLinearAttention(Part):
    """q, k (heads x head_dim) and v (heads x v_head_dim) are projections passed through an
    activation; per head the state S [head_dim, v_head_dim] follows

        S_t = decay_h S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t

    with one constant decay per head and no other scale. The heads' outputs, side by side, are
    RMS-normed together (one weight per channel), multiplied by sigmoid(gate h) channel by channel
    and projected. The state is 32-bit, starts at zero and lives in the request's state slot; the
    recurrence, its decay and the norm are computed in 32-bit in either precision.

    params: hidden, heads, head_dim, v_head_dim, decay (one number, or one per head), norm_eps,
    activation ("silu" or None); tensor names q, k, v, gate, o, norm relative to the prefix.

    One kernel walks a sequence's tokens of the step in order, whether they are a portion or a
    single token, so the result does not depend on the cut. A step that holds a long portion (256
    tokens and more of one request) cuts every portion into segments that are scanned at once and
    joined by the state that comes into each (`ops.scan_segments`): the same sums in another
    order, equal within rounding. The four projections are stacked at load into one matrix and
    read from the product's rows in place."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("hidden", "heads", "head_dim", "v_head_dim", "decay", "norm_eps", "q", "k", "v", "gate", "o", "norm")
        p = params
        self.hidden, self.heads, self.dim, self.vdim = (int(p[k]) for k in ("hidden", "heads", "head_dim", "v_head_dim"))
        if self.dim > 256:
            raise ValueError(f"head_dim up to 256 is supported, got {self.dim}")
        decay = p["decay"]
        self.decay_values = [float(d) for d in decay] if isinstance(decay, (list, tuple)) else [float(decay)] * self.heads
        if len(self.decay_values) != self.heads:
            raise ValueError(f"decay must be one number or one per head ({self.heads}), got {len(self.decay_values)}")
        self.norm_eps = float(p["norm_eps"])
        self.activation = p.get("activation", "silu")
        if self.activation not in ops.SCAN_ACTIVATIONS:
            raise ValueError(f"unsupported activation {self.activation!r}")
        self.names = {k: prefix + p[k] for k in ("q", "k", "v", "gate", "o", "norm")}
        self.w_in = self.w_o = self.norm_w = self.decay = None

    def tensor_specs(self):
        n, qk, vv = self.names, self.heads * self.dim, self.heads * self.vdim
        return [TensorSpec(n["q"], (qk, self.hidden)), TensorSpec(n["k"], (qk, self.hidden)),
                TensorSpec(n["v"], (vv, self.hidden)), TensorSpec(n["gate"], (vv, self.hidden)),
                TensorSpec(n["o"], (self.hidden, vv)), TensorSpec(n["norm"], (vv,), kind="vector", init="ones")]

    def cache_need(self):
        return StateNeed((self.heads, self.dim, self.vdim), torch.float32)

    def kernel_libraries(self, dtype):
        return ("linear_attention",)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        rows = [tensors.pop(n["q"]), tensors.pop(n["k"]), tensors.pop(n["v"]), tensors.pop(n["gate"])]
        used = sum(r.shape[0] for r in rows)
        if used % 16:           # whole 16-byte pieces per output row
            rows.append(torch.zeros((16 - used % 16, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o, self.norm_w = tensors[n["o"]], tensors[n["norm"]]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=runtime.device)

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        tokens, qk, vv = h.shape[0], self.heads * self.dim, self.heads * self.vdim
        proj = self.runtime.linear(h, self.w_in)                    # [T, q | k | v | gate (| padding)]
        scanned = torch.empty((tokens, vv), dtype=torch.float32, device=h.device)
        segment_tokens, segments = ops.scan_segments(batch.q_lens, 4 * self.heads * self.dim * self.vdim)
        scratch = torch.empty((segments, self.heads, self.dim, self.vdim), dtype=torch.float32, device=h.device) if segments else None
        ops.decay_scan(proj, 0, qk, 2 * qk, scanned, cache.state, batch.cu_q, batch.state_slots, self.decay, batch.n_seqs,
                       self.heads, self.dim, self.vdim, self.activation, segment_tokens, scratch)
        gated = torch.empty((tokens, vv), dtype=h.dtype, device=h.device)
        ops.gated_rmsnorm(scanned, proj[:, 2 * qk + vv: 2 * qk + 2 * vv], self.norm_w, self.norm_eps, gated)
        return self.runtime.linear(gated, self.w_o)


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Part):
    """Linear attention whose state is corrected towards each new value before it is read. q and k (kv_heads x
    head_dim) and v (heads x v_head_dim) are projections that pass a short causal convolution per channel
    (`taps` columns, the last one the current token's, zeros before the start) and silu; q and k heads are made
    unit vectors (x / sqrt(sum x^2 + unit_eps)), q also times head_dim^-1/2; head h reads q/k head
    h // (heads / kv_heads). Per head and token

        beta = sigmoid(W_b h),   decay = exp(-exp(A_log) * softplus(W_a h + dt_bias))
        S <- decay S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

    so the read-out sees the token's own write. Each head's o is RMS-normed over v_head_dim with one weight
    shared by the heads, multiplied by silu(W_g h) and projected. A request's state, one row of 32-bit floats in
    its state slot: S of every head, then the last taps - 1 inputs of every convolved channel.

    params: hidden, heads, kv_heads, head_dim, v_head_dim, taps, norm_eps, unit_eps (default 1e-6); tensor names
    q, k, v, q_conv, k_conv, v_conv, b, a, a_log, dt_bias, gate, norm, o relative to the prefix.

    The stacked projection leaves 32-bit rows in both precisions; convolution, unit norms, beta, decay, the
    recurrence and the norm are 32-bit arithmetic in a fixed order per token, whatever the cut or the batch."""

    NAMES = ("q", "k", "v", "q_conv", "k_conv", "v_conv", "b", "a", "a_log", "dt_bias", "gate", "norm", "o")

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("hidden", "heads", "kv_heads", "head_dim", "v_head_dim", "taps", "norm_eps", *self.NAMES)
        p = params
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim, self.taps = (
            int(p[k]) for k in ("hidden", "heads", "kv_heads", "head_dim", "v_head_dim", "taps"))
        if self.heads % self.kv_heads:
            raise ValueError(f"gated_delta_rule: heads ({self.heads}) must be a multiple of kv_heads ({self.kv_heads})")
        if self.dim > 256 or self.taps < 1:
            raise ValueError(f"gated_delta_rule: head_dim up to 256 and at least one tap, got {self.dim} and {self.taps}")
        self.norm_eps, self.unit_eps = float(p["norm_eps"]), float(p.get("unit_eps", 1e-6))
        self.names = {k: prefix + p[k] for k in self.NAMES}
        self.qk, self.vv = self.kv_heads * self.dim, self.heads * self.vdim
        self.channels = 2 * self.qk + self.vv                      # the convolved channels: q | k | v
        self.state_floats = self.heads * self.dim * self.vdim      # S of every head; the convolutions' tail follows

    def tensor_specs(self):
        n, hid = self.names, self.hidden
        return [TensorSpec(n["q"], (self.qk, hid)), TensorSpec(n["k"], (self.qk, hid)), TensorSpec(n["v"], (self.vv, hid)),
                TensorSpec(n["q_conv"], (self.qk, self.taps), kind="vector"), TensorSpec(n["k_conv"], (self.qk, self.taps), kind="vector"),
                TensorSpec(n["v_conv"], (self.vv, self.taps), kind="vector"),
                TensorSpec(n["b"], (self.heads, hid)), TensorSpec(n["a"], (self.heads, hid)),
                TensorSpec(n["a_log"], (self.heads,), kind="vector"), TensorSpec(n["dt_bias"], (self.heads,), kind="vector"),
                TensorSpec(n["gate"], (self.vv, hid)), TensorSpec(n["norm"], (self.vdim,), kind="vector", init="ones"),
                TensorSpec(n["o"], (hid, self.vv))]

    def cache_need(self):
        return StateNeed((self.state_floats + (self.taps - 1) * self.channels,), torch.float32)

    def kernel_libraries(self, dtype):
        return ("delta_rule",)

    def tile_sizes(self, dtype):
        return (ops.delta_prepare_tokens(),)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        rows = [tensors.pop(n[k]) for k in ("q", "k", "v", "gate", "b", "a")]
        used = sum(r.shape[0] for r in rows)
        if used % 16:           # whole 16-byte pieces per output row
            rows.append(torch.zeros((16 - used % 16, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()                    # [q | k | v | gate | b | a (| padding)]
        self.gate_off = self.channels
        self.b_off, self.a_off = self.channels + self.vv, self.channels + self.vv + self.heads
        self.conv = torch.cat([tensors.pop(n[k]) for k in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w, self.w_o = tensors[n["a_log"]], tensors[n["dt_bias"]], tensors[n["norm"]], tensors[n["o"]]

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        tokens = h.shape[0]
        proj = self.runtime.linear(h, self.w_in, out_dtype=torch.float32)
        prepared = torch.empty((tokens, self.channels + 2 * self.heads), dtype=torch.float32, device=h.device)
        ops.delta_prepare(proj, self.b_off, self.a_off, self.conv, self.a_log, self.dt_bias, cache.state, self.state_floats, batch,
                          prepared, self.heads, self.kv_heads, self.dim, self.vdim, self.unit_eps)
        scanned = torch.empty((tokens, self.vv), dtype=torch.float32, device=h.device)
        ops.delta_scan(prepared, scanned, cache.state, batch, self.heads, self.kv_heads, self.dim, self.vdim)
        gated = torch.empty((tokens, self.vv), dtype=h.dtype, device=h.device)
        ops.head_gated_rmsnorm(scanned, proj[:, self.gate_off: self.gate_off + self.vv], self.norm_w, self.norm_eps, gated,
                               self.heads, self.vdim)
        return self.runtime.linear(gated, self.w_o)


@register_mixer("wkv")
class TokenShiftWKV(Part):
    """Time mixing whose decay depends on the token and the key channel. With h' the input of the token before
    (zeros before a sequence's first token), each of r, k, v, g, w reads a mix of its own, h + (h' - h) * mu_s;
    r, k, v (heads x head_dim) are projections of their mixes, gate = silu(W_g mix_g), and

        w_t = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))                    per head and key channel
        o_t = (S + diag(u) k_t v_t^T)^T r_t,   S <- diag(w_t) S + k_t v_t^T     per head, S [head_dim, head_dim]

    with the bonus u for the current token only. Each head's o is divided by its root mean square, the heads side
    by side are multiplied by a weight per channel and by the gate, and projected. A request's state, one row of
    32-bit floats in its state slot: S of every head, then the previous token's input.

    params: hidden, heads, head_dim, decay_rank (rows of W_w1), norm_eps; tensor names mu_r, mu_k, mu_v, mu_g, mu_w,
    r, k, v, gate, w1, w2, w0, u, norm, o relative to the prefix.

    One kernel makes the five mixes (and moves the state's last input on), five products read one mix each and
    leave 32-bit rows, one kernel makes the decays, one walks the recurrence, one norms and gates. Decay, bonus,
    recurrence, state and the norm are 32-bit arithmetic in a fixed order per token, whatever the cut or the batch."""

    NAMES = ("mu_r", "mu_k", "mu_v", "mu_g", "mu_w", "r", "k", "v", "gate", "w1", "w2", "w0", "u", "norm", "o")

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("hidden", "heads", "head_dim", "decay_rank", "norm_eps", *self.NAMES)
        p = params
        self.hidden, self.heads, self.dim, self.rank = (int(p[k]) for k in ("hidden", "heads", "head_dim", "decay_rank"))
        if self.dim > 256:
            raise ValueError(f"wkv: head_dim up to 256 is supported, got {self.dim}")
        self.norm_eps = float(p["norm_eps"])
        self.names = {k: prefix + p[k] for k in self.NAMES}
        self.channels = self.heads * self.dim
        self.state_floats = self.heads * self.dim * self.dim       # S of every head; the previous input follows

    def tensor_specs(self):
        n, hid, ch = self.names, self.hidden, self.channels
        return [*(TensorSpec(n["mu_" + s], (hid,), kind="vector") for s in "rkvgw"),
                TensorSpec(n["r"], (ch, hid)), TensorSpec(n["k"], (ch, hid)), TensorSpec(n["v"], (ch, hid)),
                TensorSpec(n["gate"], (ch, hid)), TensorSpec(n["w1"], (self.rank, hid)), TensorSpec(n["w2"], (ch, self.rank)),
                TensorSpec(n["w0"], (ch,), kind="vector"), TensorSpec(n["u"], (self.heads, self.dim), kind="vector"),
                TensorSpec(n["norm"], (ch,), kind="vector", init="ones"), TensorSpec(n["o"], (hid, ch))]

    def cache_need(self):
        return StateNeed((self.state_floats + self.hidden,), torch.float32)

    def kernel_libraries(self, dtype):
        return ("wkv", "delta_rule")

    def tile_sizes(self, dtype):
        return (ops.wkv_mix_tokens(),)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        self.mu = torch.stack([tensors.pop(n["mu_" + s]) for s in "rkvgw"]).contiguous()       # [5, hidden], 32-bit
        self.w_in = [tensors[n[k]] for k in ("r", "k", "v", "gate")]
        w1 = tensors.pop(n["w1"])
        if self.rank % 16:      # whole 16-byte pieces per output row
            w1 = torch.cat((w1, torch.zeros((16 - self.rank % 16, self.hidden), dtype=w1.dtype, device=w1.device)), dim=0)
        self.w1 = w1.contiguous()
        self.w2, self.w0, self.u = tensors[n["w2"]], tensors[n["w0"]], tensors[n["u"]]
        self.norm_w, self.w_o = tensors[n["norm"]], tensors[n["o"]]
        self._product = ops.gemm_simt if runtime.dtype == torch.float32 else ops.gemm_bf16

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        tokens, ch = h.shape[0], self.channels
        mixes = torch.empty((5, tokens, self.hidden), dtype=h.dtype, device=h.device)
        ops.wkv_shift_mix(h, self.mu, cache.state, self.state_floats, batch, mixes)
        proj = torch.empty((tokens, 4 * ch), dtype=torch.float32, device=h.device)             # [r | k | v | gate]
        for index, weight in enumerate(self.w_in):
            self._product(mixes[index], weight, proj[:, index * ch: (index + 1) * ch])
        lora = torch.empty((tokens, self.w1.shape[0]), dtype=torch.float32, device=h.device)
        self._product(mixes[4], self.w1, lora)
        decay = torch.empty((tokens, ch), dtype=torch.float32, device=h.device)
        ops.wkv_decay(lora, self.w2, self.w0, decay)
        scanned = torch.empty((tokens, ch), dtype=torch.float32, device=h.device)
        ops.wkv_scan(proj[:, :ch], proj[:, ch: 2 * ch], proj[:, 2 * ch: 3 * ch], decay, self.u, scanned, cache.state, batch,
                     self.heads, self.dim)
        gated = torch.empty((tokens, ch), dtype=h.dtype, device=h.device)
        ops.head_gated_rmsnorm(scanned, proj[:, 3 * ch:], self.norm_w, self.norm_eps, gated, self.heads, self.dim)
        return self.runtime.linear(gated, self.w_o)
