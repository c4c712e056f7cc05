"""A Nemotron-H-shaped hybrid model in torch, random-init: TEST AND BENCHMARK STAND-IN, not product code.

It stands in for the HuggingFace remote-code module the reference patches (the checkpoint, its modeling
file, ``mamba_ssm`` and ``causal_conv1d`` are not available offline).  It loads the way the real one does,
``AutoModelForCausalLM.from_pretrained(<this directory>, trust_remote_code=True)``, and has what the
reference's scripts and patch functions reach for: the block layout
(``backbone.layers[i].{block_type, norm, mixer, residual_in_fp32}``), the attribute names on the mixers,
module-global ``selective_state_update`` and ``repeat_kv``, a ``HybridMambaAttentionDynamicCache`` with
``conv_states`` / ``ssm_states`` lists, ``config.hybrid_override_pattern`` and ``config.conv_kernel``.
The Mamba2 step follows the public Mamba2 formulation (in_proj -> causal conv1d update -> selective state
update -> gated RMSNorm -> out_proj), attention has no RoPE, the MLP is squared-ReLU.  On CUDA the two
unquantised steps go through the library's baselines (``layer_quant_b200.dense_state``), the stand-ins for
the third-party kernels the real module imports; on CPU they are plain torch.
"""
from __future__ import annotations

from types import SimpleNamespace

import torch
import torch.nn as nn
import torch.nn.functional as F
from transformers import PreTrainedModel

from .configuration_nemotron_h_shim import NemotronHShimConfig, nemotron_h_8b_config, tiny_config  # noqa: F401


def repeat_kv(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    b, h, t, d = hidden_states.shape
    if n_rep == 1:
        return hidden_states
    return hidden_states[:, :, None].expand(b, h, n_rep, t, d).reshape(b, h * n_rep, t, d)


def selective_state_update(ssm_state, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False):
    """Unquantised decode step on a floating-point state [B, H, P, N] (updated in place), fp32 math:
    the baseline the MX kernels are compared with (and the module-global symbol their patch replaces)."""
    if ssm_state.is_cuda and z is None:
        from layer_quant_b200 import dense_state
        return dense_state.selective_state_update(ssm_state, x, dt, A, B, C, D=D, dt_bias=dt_bias, dt_softplus=dt_softplus)
    return selective_state_update_torch(ssm_state, x, dt, A, B, C, D=D, z=z, dt_bias=dt_bias, dt_softplus=dt_softplus)


def selective_state_update_torch(ssm_state, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False):
    batch, nheads, dim, dstate = ssm_state.shape
    dt = dt.float()
    if dt_bias is not None:
        dt = dt + dt_bias.float()
    if dt_softplus:
        dt = F.softplus(dt)
    ratio = nheads // B.shape[1]
    Bh = B.float().repeat_interleave(ratio, dim=1)[:, :, None, :]
    Ch = C.float().repeat_interleave(ratio, dim=1)[:, :, None, :]
    dA = torch.exp(A.float()[None] * dt[..., None])
    h = ssm_state.float() * dA + Bh * dt[..., None] * x.float()[..., None]
    ssm_state.copy_(h.to(ssm_state.dtype))
    y = (h * Ch).sum(-1)
    if D is not None:
        y = y + x.float() * D.float()
    if z is not None:
        y = y * z.float()
    return y.to(x.dtype)


class HybridMambaAttentionDynamicCache:
    def __init__(self, config, batch_size, dtype=torch.bfloat16, device=None):
        self.conv_states, self.ssm_states = [], []
        conv_dim = config.mamba_intermediate + 2 * config.n_groups * config.ssm_state_size
        for kind in config.hybrid_override_pattern:
            if kind == "M":
                self.conv_states.append(torch.zeros(batch_size, conv_dim, config.conv_kernel, device=device, dtype=dtype))
                self.ssm_states.append(torch.zeros(batch_size, config.mamba_num_heads, config.mamba_head_dim,
                                                   config.ssm_state_size, device=device, dtype=dtype))
            else:
                self.conv_states.append(torch.zeros(batch_size, 0, device=device, dtype=dtype))
                self.ssm_states.append(torch.zeros(batch_size, 0, device=device, dtype=dtype))
        self.key_cache = [None] * len(config.hybrid_override_pattern)  # bf16 KV of the unpatched attention
        self.value_cache = [None] * len(config.hybrid_override_pattern)
        self.static_kv_len = 0  # > 0: key / value caches are pre-sized [B, Hkv, static_kv_len, D] and written in place

    def presize_kv(self, max_len: int) -> None:
        """Switch the unpatched attention to pre-sized K / V buffers of ``max_len`` rows (rows already cached are
        kept): single-token steps then write row ``cache_position`` in place and attend under a length mask, so a
        step allocates nothing and can be recorded in a CUDA graph."""
        for i, k in enumerate(self.key_cache):
            if k is None:
                continue
            v = self.value_cache[i]
            nk, nv = k.new_zeros(k.shape[0], k.shape[1], max_len, k.shape[3]), v.new_zeros(v.shape[0], v.shape[1], max_len, v.shape[3])
            nk[:, :, :k.shape[2]], nv[:, :, :v.shape[2]] = k, v
            self.key_cache[i], self.value_cache[i] = nk, nv
        self.static_kv_len = max_len


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x, gate=None):
        if gate is not None:
            x = x * F.silu(gate)
        return F.rms_norm(x.to(self.weight.dtype), (self.weight.shape[0],), self.weight, self.eps)


class Mamba2Mixer(nn.Module):
    def __init__(self, config, layer_idx):
        super().__init__()
        self.layer_idx = layer_idx
        self.num_heads, self.head_dim = config.mamba_num_heads, config.mamba_head_dim
        self.ssm_state_size, self.n_groups = config.ssm_state_size, config.n_groups
        self.intermediate_size = config.mamba_intermediate
        self.conv_dim = self.intermediate_size + 2 * self.n_groups * self.ssm_state_size
        self.conv_kernel_size = config.conv_kernel
        self.in_proj = nn.Linear(config.hidden_size, self.intermediate_size + self.conv_dim + self.num_heads, bias=False)
        self.conv1d = nn.Conv1d(self.conv_dim, self.conv_dim, config.conv_kernel, groups=self.conv_dim, padding=config.conv_kernel - 1)
        self.dt_bias = nn.Parameter(torch.rand(self.num_heads) * 2.0 - 4.0)
        self.A_log = nn.Parameter(torch.log(torch.rand(self.num_heads) * 15.0 + 1.0))
        self.D = nn.Parameter(torch.rand(self.num_heads))
        self.norm = RMSNorm(self.intermediate_size)
        self.out_proj = nn.Linear(self.intermediate_size, config.hidden_size, bias=False)

    def _step(self, hs, cache_params):
        """hs [B, hidden] -> [B, hidden]; one token through conv state and SSM state."""
        import sys
        module = sys.modules[__name__]
        batch = hs.shape[0]
        gate, xbc, dt = self.in_proj(hs).split([self.intermediate_size, self.conv_dim, self.num_heads], dim=-1)
        conv_state = cache_params.conv_states[self.layer_idx]
        if hs.is_cuda:
            from layer_quant_b200 import dense_state
            xbc = dense_state.causal_conv1d_update(xbc, conv_state, self.conv1d.weight.squeeze(1), self.conv1d.bias, "silu")
        else:
            conv_state.copy_(torch.roll(conv_state, shifts=-1, dims=-1))
            conv_state[:, :, -1] = xbc
            xbc = F.silu((conv_state.float() * self.conv1d.weight.squeeze(1).float()).sum(-1) + self.conv1d.bias.float()).to(hs.dtype)
        x, B, C = xbc.split([self.intermediate_size, self.n_groups * self.ssm_state_size, self.n_groups * self.ssm_state_size], dim=-1)
        A = (-torch.exp(self.A_log.float()))[:, None, None].expand(-1, self.head_dim, self.ssm_state_size)  # stride-0 view
        y = module.selective_state_update(  # looked up at call time: this is the symbol the MX patch replaces
            cache_params.ssm_states[self.layer_idx], x.reshape(batch, self.num_heads, self.head_dim),
            dt[:, :, None].expand(-1, -1, self.head_dim), A, B.view(batch, self.n_groups, -1), C.view(batch, self.n_groups, -1),
            self.D[:, None].expand(-1, self.head_dim), z=None, dt_bias=self.dt_bias[:, None].expand(-1, self.head_dim),
            dt_softplus=True)
        return self.out_proj(self.norm(y.reshape(batch, -1), gate))

    def forward(self, hidden_states, cache_params=None, cache_position=None, attention_mask=None):
        t_len = hidden_states.shape[1]
        if t_len == 1:
            return self._step(hidden_states[:, 0], cache_params).unsqueeze(1)
        # Several tokens (a prompt): the projections, the convolution and the gated norm run over the whole sequence at
        # once; only the state recurrence itself goes token by token through the same update the decode step uses.
        import sys
        module = sys.modules[__name__]
        batch = hidden_states.shape[0]
        gate, xbc, dt = self.in_proj(hidden_states).split([self.intermediate_size, self.conv_dim, self.num_heads], dim=-1)
        conv_state = cache_params.conv_states[self.layer_idx]
        full = torch.cat([conv_state, xbc.transpose(1, 2).to(conv_state.dtype)], dim=2)  # [B, C, W + T]
        conv_state.copy_(full[:, :, -self.conv_kernel_size:])
        windows = full[:, :, 1:].unfold(2, self.conv_kernel_size, 1)  # [B, C, T, W]: the window ending at each token
        xbc = F.silu((windows.float() * self.conv1d.weight.squeeze(1).float()[None, :, None, :]).sum(-1)
                     + self.conv1d.bias.float()[None, :, None]).to(hidden_states.dtype).transpose(1, 2)
        x, B, C = xbc.split([self.intermediate_size, self.n_groups * self.ssm_state_size, self.n_groups * self.ssm_state_size], dim=-1)
        A = (-torch.exp(self.A_log.float()))[:, None, None].expand(-1, self.head_dim, self.ssm_state_size)
        D, bias = self.D[:, None].expand(-1, self.head_dim), self.dt_bias[:, None].expand(-1, self.head_dim)
        state = cache_params.ssm_states[self.layer_idx]
        ys = []
        for t in range(t_len):
            ys.append(module.selective_state_update(
                state, x[:, t].reshape(batch, self.num_heads, self.head_dim), dt[:, t, :, None].expand(-1, -1, self.head_dim), A,
                B[:, t].reshape(batch, self.n_groups, -1), C[:, t].reshape(batch, self.n_groups, -1), D, z=None, dt_bias=bias,
                dt_softplus=True))
        y = torch.stack(ys, dim=1).reshape(batch, t_len, -1)
        return self.out_proj(self.norm(y, gate))


class Attention(nn.Module):
    def __init__(self, config, layer_idx):
        super().__init__()
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads, self.num_key_value_heads, self.head_dim = config.num_attention_heads, config.num_key_value_heads, config.head_dim
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.attention_dropout = 0.0
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=False)
        self.k_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=False)
        self.v_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=False)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, self.hidden_size, bias=False)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None, output_attentions=False,
                use_cache=False, cache_position=None):
        """Unquantised reference path: bf16 K/V appended to past_key_value.key_cache / value_cache."""
        b, t, _ = hidden_states.shape
        q = self.q_proj(hidden_states).view(b, t, self.num_heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(hidden_states).view(b, t, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(hidden_states).view(b, t, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        static = past_key_value is not None and getattr(past_key_value, "static_kv_len", 0) > 0 and t == 1
        if static:
            # pre-sized buffers: write row cache_position in place, attend all rows under a length mask (no allocation,
            # no host read of the position: the step can be recorded in a CUDA graph)
            pk, pv = past_key_value.key_cache[self.layer_idx], past_key_value.value_cache[self.layer_idx]
            pos = cache_position.to(device=k.device, dtype=torch.long).reshape(1)
            pk.index_copy_(2, pos, k)
            pv.index_copy_(2, pos, v)
            g = self.num_key_value_groups
            qg = q.reshape(b, self.num_key_value_heads, g, self.head_dim)
            scores = torch.einsum("bkgd,bktd->bkgt", qg, pk).float() * (self.head_dim ** -0.5)
            hidden = torch.arange(pk.shape[2], device=k.device) > pos
            probs = torch.softmax(scores.masked_fill(hidden, float("-inf")), dim=-1).to(pv.dtype)
            out = torch.einsum("bkgt,bktd->bkgd", probs, pv).reshape(b, self.num_heads, 1, self.head_dim)
            return self.o_proj(out.transpose(1, 2).reshape(b, t, -1)), None, past_key_value
        if past_key_value is not None:
            pk, pv = past_key_value.key_cache[self.layer_idx], past_key_value.value_cache[self.layer_idx]
            if pk is not None:
                k, v = torch.cat([pk, k], dim=2), torch.cat([pv, v], dim=2)
            past_key_value.key_cache[self.layer_idx], past_key_value.value_cache[self.layer_idx] = k, v
        if t == 1:
            # one query token: grouped matmuls with an fp32 softmax (torch's fused attention costs tens of
            # milliseconds of host time per call for this shape on some builds)
            g = self.num_key_value_groups
            qg = q.reshape(b, self.num_key_value_heads, g, self.head_dim)
            scores = torch.einsum("bkgd,bktd->bkgt", qg, k).float() * (self.head_dim ** -0.5)
            probs = torch.softmax(scores, dim=-1).to(v.dtype)
            out = torch.einsum("bkgt,bktd->bkgd", probs, v).reshape(b, self.num_heads, 1, self.head_dim)
        else:
            out = F.scaled_dot_product_attention(q, repeat_kv(k, self.num_key_value_groups), repeat_kv(v, self.num_key_value_groups),
                                                 is_causal=True)
        return self.o_proj(out.transpose(1, 2).reshape(b, t, -1)), None, past_key_value


class MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.relu(self.up_proj(x)).square())


class Block(nn.Module):
    def __init__(self, config, layer_idx, kind):
        super().__init__()
        self.block_type = {"M": "mamba", "*": "attention", "-": "mlp"}[kind]
        self.residual_in_fp32 = False
        self.norm = RMSNorm(config.hidden_size)
        self.mixer = {"M": lambda: Mamba2Mixer(config, layer_idx), "*": lambda: Attention(config, layer_idx), "-": lambda: MLP(config)}[kind]()

    def forward(self, hidden_states, cache_params=None, cache_position=None, attention_mask=None):
        residual = hidden_states
        hidden_states = self.norm(hidden_states.to(dtype=self.norm.weight.dtype))
        if self.block_type == "mamba":
            hidden_states = self.mixer(hidden_states, cache_params=cache_params, cache_position=cache_position)
        elif self.block_type == "attention":
            hidden_states = self.mixer(hidden_states, attention_mask=attention_mask, past_key_value=cache_params,
                                       use_cache=cache_params is not None, cache_position=cache_position)[0]
        else:
            hidden_states = self.mixer(hidden_states)
        return residual + hidden_states


class NemotronHShimPreTrainedModel(PreTrainedModel):
    config_class = NemotronHShimConfig
    base_model_prefix = "backbone"
    _no_split_modules = ["Block"]

    def _init_weights(self, module):
        std = self.config.initializer_range
        if isinstance(module, (nn.Linear, nn.Conv1d)):
            nn.init.normal_(module.weight, mean=0.0, std=std)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, mean=0.0, std=std)


class NemotronHShimForCausalLM(NemotronHShimPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.backbone = nn.Module()
        self.backbone.embeddings = nn.Embedding(config.vocab_size, config.hidden_size)
        self.backbone.layers = nn.ModuleList(Block(config, i, k) for i, k in enumerate(config.hybrid_override_pattern))
        self.backbone.norm_f = RMSNorm(config.hidden_size)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def forward(self, input_ids, cache_params=None, cache_position=None, use_cache=True, return_dict=True, attention_mask=None,
                logits_to_keep=0, **kwargs):
        h = self.backbone.embeddings(input_ids)
        for layer in self.backbone.layers:
            h = layer(h, cache_params=cache_params, cache_position=cache_position, attention_mask=attention_mask)
        if logits_to_keep:
            h = h[:, -logits_to_keep:]
        return SimpleNamespace(logits=self.lm_head(self.backbone.norm_f(h)))
