"""RWKV-7 ("Goose"): an attention-free recurrent language model.

Every block has a time-mix (a generalised delta rule over a per-head N x N state with per-channel
decay, in-context learning rate `a` and removal key `kk`) and a channel-mix (squared-ReLU MLP), both fed
through a token shift (the previous token's activation).  There is no KV cache: a running sequence owns
one state slot holding, per layer, the two shift vectors and the [heads, N, N] fp32 state; the engine's
slot bookkeeping is the one of the other recurrent-state models.

    w      = exp(-exp(logsigmoid(w0 + tanh(xw W1) W2) - 0.5))            per-channel decay in (0, 1)
    a      = sigmoid(a0 + (xa A1) A2)                                     in-context learning rate
    kk     = normalize(k * k_k) per head ;  k' = k * (1 + (a - 1) * k_a)
    v      = v + (v_first - v) * sigmoid(v0 + (xv V1) V2)                 (layers > 0: value residual)
    S_t    = S_{t-1} diag(w) - S_{t-1} kk^T (kk * a) + v^T k'             per head
    y_t    = S_t r ;  out = W_o((groupnorm(y) + (r . k' . r_k) v) * g),  g = sigmoid(xg G1) G2

Parity: xllm/models/llm/rwkv7.h and core/layers/rwkv7_decoder_layer.cpp (parameter names `emb`,
`blocks.N.{ln0,ln1,ln2,att.*,ffn.*}`, `ln_out`, `head`, the RWKV-LM checkpoint layout; the RWKV "world"
trie tokenizer is utils/tokenizer_extra.py).  The recurrence runs in tensor ops per token; a chunked
kernel for it is not built.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .layers import LMHead, Linear, Module, VocabEmbedding
from .registry import register_model
from ..parallel.state import single


class _LayerNorm(Module):
    def __init__(self, dim, eps, dtype, device):
        super().__init__()
        self.eps = eps
        self.weight = self.add_param("weight", torch.ones(dim, dtype=dtype, device=device))
        self.bias = self.add_param("bias", torch.zeros(dim, dtype=dtype, device=device))

    def forward(self, x):
        return F.layer_norm(x.float(), (x.shape[-1],), self.weight.float(), self.bias.float(), self.eps).to(x.dtype)

    __call__ = forward


class Rwkv7State:
    """Per running sequence: shift vectors of both mixers and the wkv state of every layer."""

    def __init__(self, n_layers, slots, hidden, heads, head_size, device, dtype):
        self.att_shift = torch.zeros(n_layers, slots, hidden, dtype=dtype, device=device)
        self.ffn_shift = torch.zeros(n_layers, slots, hidden, dtype=dtype, device=device)
        self.wkv = torch.zeros(n_layers, slots, heads, head_size, head_size, dtype=torch.float32, device=device)
        self.free = list(range(slots - 1, -1, -1))
        self.owner = {}
        self.n_slots = slots

    def slot_of(self, seq_id):
        s = self.owner.get(seq_id)
        if s is None:
            if not self.free:
                raise RuntimeError("no free state slot: the scheduler admitted more sequences than the pool holds")
            s = self.owner[seq_id] = self.free.pop()
        return s

    def release(self, seq_id):
        s = self.owner.pop(seq_id, None)
        if s is not None:
            self.free.append(s)


class TimeMix(Module):
    def __init__(self, args, idx, dtype, device):
        super().__init__()
        C, H, N = args.hidden_size, args.num_attention_heads, args.head_dim
        self.C, self.H, self.N, self.idx = C, H, N, idx
        e = args.extra
        z = lambda *s: torch.zeros(*s, dtype=dtype, device=device)
        for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g", "w0", "a0", "v0"):
            setattr(self, n, self.add_param(n, z(1, 1, C)))
        self.k_k = self.add_param("k_k", torch.ones(1, 1, C, dtype=dtype, device=device))
        self.k_a = self.add_param("k_a", torch.ones(1, 1, C, dtype=dtype, device=device))
        self.r_k = self.add_param("r_k", z(H, N))
        for n, rank in (("w", e.get("decay_low_rank_dim", 64)), ("a", e.get("a_low_rank_dim", 64)),
                        ("v", e.get("v_low_rank_dim", 32)), ("g", e.get("gate_low_rank_dim", 128))):
            if n == "v" and idx == 0:
                continue                                   # the first layer defines v_first and has no value residual
            setattr(self, n + "1", self.add_param(n + "1", z(C, rank)))
            setattr(self, n + "2", self.add_param(n + "2", z(rank, C)))
        self.receptance = self.add_module("receptance", Linear(C, C, False, dtype, device))
        self.key = self.add_module("key", Linear(C, C, False, dtype, device))
        self.value = self.add_module("value", Linear(C, C, False, dtype, device))
        self.output = self.add_module("output", Linear(C, C, False, dtype, device))
        self.ln_x_w = self.add_param("ln_x.weight", torch.ones(C, dtype=dtype, device=device))
        self.ln_x_b = self.add_param("ln_x.bias", z(C))
        self.gn_eps = float(e.get("group_norm_eps", 64e-5))

    def forward(self, x, shift_in, S, v_first):
        """x [T, C] of ONE sequence; shift_in [C] (previous token's input, zeros at position 0); S [H, N, N]
        fp32.  Returns (out [T, C], last input [C], S', v_first [T, C])."""
        T, C, H, N = x.shape[0], self.C, self.H, self.N
        prev = torch.cat([shift_in[None].to(x.dtype), x[:-1]], 0)
        xx = prev - x
        mix = lambda c: x + xx * c.view(C)
        xr, xw, xk, xv, xa, xg = (mix(c) for c in (self.x_r, self.x_w, self.x_k, self.x_v, self.x_a, self.x_g))
        r, k, v = self.receptance(xr), self.key(xk), self.value(xv)
        f = lambda t: t.float()
        w = torch.exp(-torch.exp(F.logsigmoid(f(self.w0).view(C) + torch.tanh(f(xw) @ f(self.w1)) @ f(self.w2)) - 0.5))
        a = torch.sigmoid(f(self.a0).view(C) + (f(xa) @ f(self.a1)) @ f(self.a2))
        g = torch.sigmoid(f(xg) @ f(self.g1)) @ f(self.g2)
        rf, kf, vf = f(r).view(T, H, N), f(k).view(T, H, N), f(v).view(T, H, N)
        ah = a.view(T, H, N)
        kk = F.normalize(kf * f(self.k_k).view(1, H, N), dim=-1, p=2.0)
        k2 = kf * (1.0 + (ah - 1.0) * f(self.k_a).view(1, H, N))
        if self.idx == 0:
            v_first = v
        else:
            blend = torch.sigmoid(f(self.v0).view(C) + (f(xv) @ f(self.v1)) @ f(self.v2)).view(T, H, N)
            vf = vf + (f(v_first).view(T, H, N) - vf) * blend
        wh = w.view(T, H, N)
        y = torch.empty(T, H, N, dtype=torch.float32, device=x.device)
        S = S.clone()
        for t in range(T):
            ab = (-kk[t])[:, :, None] * (kk[t] * ah[t])[:, None, :]              # [H, N, N]
            S = S * wh[t][:, None, :] + torch.bmm(S, ab) + vf[t][:, :, None] * k2[t][:, None, :]
            y[t] = torch.bmm(S, rf[t][:, :, None])[:, :, 0]
        yn = F.group_norm(y.view(T, C), H, f(self.ln_x_w), f(self.ln_x_b), self.gn_eps)
        rk = (rf * k2 * f(self.r_k)[None]).sum(-1, keepdim=True)
        out = self.output(((yn + (rk * vf).view(T, C)) * g).to(x.dtype))
        return out, x[-1], S, v_first

    __call__ = forward


class ChannelMix(Module):
    def __init__(self, args, dtype, device):
        super().__init__()
        C, I = args.hidden_size, args.intermediate_size
        self.x_k = self.add_param("x_k", torch.zeros(1, 1, C, dtype=dtype, device=device))
        self.key = self.add_module("key", Linear(C, I, False, dtype, device))
        self.value = self.add_module("value", Linear(I, C, False, dtype, device))

    def forward(self, x, shift_in):
        prev = torch.cat([shift_in[None].to(x.dtype), x[:-1]], 0)
        k = x + (prev - x) * self.x_k.view(-1)
        return self.value(torch.relu(self.key(k)) ** 2), x[-1]

    __call__ = forward


class Rwkv7Block(Module):
    def __init__(self, args, idx, dtype, device):
        super().__init__()
        eps = float(args.extra.get("layer_norm_eps", 1e-5))
        C = args.hidden_size
        self.idx = idx
        self.ln0 = self.add_module("ln0", _LayerNorm(C, eps, dtype, device)) if idx == 0 else None
        self.ln1 = self.add_module("ln1", _LayerNorm(C, eps, dtype, device))
        self.ln2 = self.add_module("ln2", _LayerNorm(C, eps, dtype, device))
        self.att = self.add_module("att", TimeMix(args, idx, dtype, device))
        self.ffn = self.add_module("ffn", ChannelMix(args, dtype, device))


class Rwkv7CausalLM(Module):
    needs_state = True
    supports_graph = False
    supports_prefill_graph = False
    fused_tp = False
    kv_planes = 1
    num_kv_heads_local = 1          # the paged KV cache is unused: the smallest legal geometry
    head_dim = 64

    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps=None):
        super().__init__()
        self.args, self.ps, self.dtype, self.device = args, ps or single(), dtype, torch.device(device)
        assert self.ps.tp_size == 1, "RWKV-7 runs unsharded"
        C = args.hidden_size
        self.embed = self.add_module("emb", VocabEmbedding(args.vocab_size, C, dtype, device, self.ps))
        blocks = Module()
        self.add_module("blocks", blocks)
        self.layers = [blocks.add_module(str(i), Rwkv7Block(args, i, dtype, device)) for i in range(args.num_hidden_layers)]
        self.ln_out = self.add_module("ln_out", _LayerNorm(C, float(args.extra.get("layer_norm_eps", 1e-5)), dtype, device))
        self.lm_head = LMHead(args.vocab_size, C, dtype, device, self.ps, tied=None)
        self.add_module("head", self.lm_head)
        self.state = None

    def alloc_state(self, slots):
        a = self.args
        self.state = Rwkv7State(a.num_hidden_layers, slots, a.hidden_size, a.num_attention_heads, a.head_dim, self.device,
                                self.dtype)
        return self.state

    @staticmethod
    def remap_weight(name, w):
        # RWKV-LM checkpoints have no `model.` prefix; exports from wrappers do
        if name.startswith("model."):
            name = name[len("model."):]
        return [(name, w)]

    def init_random(self, std=0.02, seed=0):
        super().init_random(std, seed)
        g = torch.Generator().manual_seed(seed + 1)
        for name, t in self.named_params():
            if name.endswith(("ln0.weight", "ln1.weight", "ln2.weight", "ln_out.weight", "ln_x.weight", "k_k", "k_a")):
                t.fill_(1.0)
            elif name.endswith(".bias") or name.endswith(("w0", "a0", "v0")):
                t.zero_()
            elif name.endswith(("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")):
                t.copy_(torch.rand(t.shape, generator=g).to(t.dtype))
            elif name.endswith(("w1", "w2", "a1", "a2", "v1", "v2", "g1", "g2", "r_k")):
                t.copy_((torch.randn(t.shape, generator=g) * 0.1).to(t.dtype))

    def forward(self, tokens, positions, meta, kv_caches, embeds=None):
        st = self.state
        x = self.embed(tokens)
        slots, fresh, bounds = meta.state_slots.tolist(), meta.state_fresh, meta.seq_bounds
        out = torch.empty_like(x)
        for s, (a, b) in enumerate(bounds):
            if b <= a:
                continue
            slot = slots[s]
            if fresh[s]:
                st.att_shift[:, slot].zero_()
                st.ffn_shift[:, slot].zero_()
                st.wkv[:, slot].zero_()
            h = x[a:b]
            v_first = None
            for li, blk in enumerate(self.layers):
                if blk.ln0 is not None:
                    h = blk.ln0(h)
                y, last, S, v_first = blk.att(blk.ln1(h), st.att_shift[li, slot], st.wkv[li, slot], v_first)
                st.att_shift[li, slot] = last
                st.wkv[li, slot] = S
                h = h + y
                y, last = blk.ffn(blk.ln2(h), st.ffn_shift[li, slot])
                st.ffn_shift[li, slot] = last
                h = h + y
            out[a:b] = h
        return self.ln_out(out)

    def logits(self, hidden_rows):
        return self.lm_head(hidden_rows)

    def logits_local(self, hidden_rows):
        return self.lm_head.forward_local(hidden_rows)

    def gather_logits(self, local):
        return self.lm_head.gather(local)

    def greedy_from_local(self, local):
        return self.lm_head.greedy_from_local(local)

    __call__ = forward


@register_model("rwkv7", "RWKV7ForCausalLM", "Rwkv7ForCausalLM")
def build_rwkv7(args, dtype, device, ps):
    return Rwkv7CausalLM(args, dtype, device, ps)
