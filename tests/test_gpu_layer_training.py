"""Whole-model regression on the GPU: a small language model whose mixer layers follow the reference layer's
forward (palimpsa/layers/palimpsa.py:262-345, without the short convolution) is trained twice from the same
initial weights on the same seeded token stream -- once with the fused kernels of this package
(layer_prologue -> chunk_palimpsa -> layer_epilogue), once with the layer's own eager lines around the
naive recurrence -- and the two loss curves must coincide.  Exercises every backward under a real optimizer."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from tests.gpu_util import DEV

pytestmark = pytest.mark.gpu


class Mixer(nn.Module):
    def __init__(self, d_model, H, K, V, fused):
        super().__init__()
        self.H, self.K, self.V, self.fused = H, K, V, fused
        self.q_proj, self.k_proj = nn.Linear(d_model, H * K, bias=False), nn.Linear(d_model, H * K, bias=False)
        self.v_proj, self.g_proj = nn.Linear(d_model, H * V, bias=False), nn.Linear(d_model, H * V, bias=False)
        self.b_proj = nn.Linear(d_model, H * V, bias=False)
        self.dt_proj, self.bs_proj = nn.Linear(d_model, H, bias=False), nn.Linear(d_model, H, bias=False)
        self.o_proj = nn.Linear(H * V, d_model, bias=False)
        self.dt_bias = nn.Parameter(torch.linspace(-2.0, 0.0, H))
        self.b_scale = nn.Parameter(torch.ones(H))
        self.A_log = nn.Parameter(torch.zeros(H))
        self.Ip_log = nn.Parameter(torch.zeros(H), requires_grad=False)
        self.D = nn.Parameter(torch.ones(H))
        self.norm_weight = nn.Parameter(torch.ones(V))

    def forward(self, h):
        B, T, _ = h.shape
        H, K, V = self.H, self.K, self.V
        q = F.silu(self.q_proj(h)).view(B, T, H, K)
        k = F.silu(self.k_proj(h)).view(B, T, H, K)
        x = F.silu(self.v_proj(h)).view(B, T, H, V)
        b_raw = self.b_proj(h).view(B, T, H, V)
        gate = self.g_proj(h).view(B, T, H, V)
        dt_raw, bs_raw = self.dt_proj(h), self.bs_proj(h)
        A, Ip = self.A_log.float().exp(), self.Ip_log.float().exp()
        if self.fused:
            from palimpsa_b200.layers import layer_epilogue, layer_prologue
            from palimpsa_b200.ops import chunk_palimpsa
            q, k, v, b, dt = layer_prologue(q, k, x, b_raw, dt_raw, bs_raw, self.dt_bias, self.b_scale)
            o = chunk_palimpsa(q, k, v, b, dt, A, Ip, chunk_size=16)
            o = layer_epilogue(o, x, self.D, self.norm_weight, gate, eps=1e-5)
        else:
            from palimpsa_b200.ops import palimpsa_ref
            dt = F.softplus(dt_raw.float() + self.dt_bias)
            q, k = F.normalize(q, p=2, dim=-1), F.normalize(k, p=2, dim=-1)
            bs = torch.sigmoid(bs_raw.float()).to(h.dtype)
            v = x * bs.unsqueeze(-1)
            b = torch.sigmoid(b_raw.float()) * F.softplus(self.b_scale.view(1, 1, -1, 1).float())
            b = (b * bs.unsqueeze(-1)).to(h.dtype)
            o = palimpsa_ref(q, k, v, b, dt, A, Ip)
            o = o + x * self.D[None, None, :, None]
            o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-5) * self.norm_weight
            o = o * gate * torch.sigmoid(gate)
        return self.o_proj(o.reshape(B, T, H * V))


class TinyLM(nn.Module):
    def __init__(self, fused, vocab=64, d_model=64, layers=2, H=2, K=32, V=32):
        super().__init__()
        self.emb = nn.Embedding(vocab, d_model)
        self.mixers = nn.ModuleList([Mixer(d_model, H, K, V, fused) for _ in range(layers)])
        self.mlps = nn.ModuleList([nn.Sequential(nn.Linear(d_model, 2 * d_model), nn.GELU(),
                                                 nn.Linear(2 * d_model, d_model)) for _ in range(layers)])
        self.head = nn.Linear(d_model, vocab, bias=False)

    def forward(self, idx):
        h = self.emb(idx)
        for mix, mlp in zip(self.mixers, self.mlps):
            h = h + mix(F.rms_norm(h, (h.shape[-1],)))
            h = h + mlp(F.rms_norm(h, (h.shape[-1],)))
        return self.head(h)


def _train(fused, state, data, steps):
    torch.manual_seed(0)
    model = TinyLM(fused).to(DEV)
    model.load_state_dict(state)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.0)
    losses = []
    for s in range(steps):
        idx = data[s]
        logits = model(idx[:, :-1])
        loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), idx[:, 1:].reshape(-1))
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses


def test_loss_curves_of_fused_and_eager_models_coincide():
    torch.manual_seed(123)
    state = {k: v.clone() for k, v in TinyLM(False).state_dict().items()}
    gen = torch.Generator().manual_seed(5)
    steps = 12
    # a learnable stream: tokens follow a fixed random permutation cycle with some noise
    perm = torch.randperm(64, generator=gen)
    data = []
    for _ in range(steps):
        start = torch.randint(0, 64, (4, 1), generator=gen)
        seq = [start]
        for _ in range(48):
            nxt = perm[seq[-1]]
            noise = torch.randint(0, 64, nxt.shape, generator=gen)
            seq.append(torch.where(torch.rand(nxt.shape, generator=gen) < 0.1, noise, nxt))
        data.append(torch.cat(seq, 1).to(DEV))
    eager = _train(False, state, data, steps)
    fused = _train(True, state, data, steps)
    assert eager[-1] < eager[0] - 0.2, f"the model did not learn: {eager}"
    for s, (a, b) in enumerate(zip(eager, fused)):
        assert abs(a - b) <= 2e-3 * max(1.0, abs(a)), f"step {s}: eager {a:.6f} vs fused {b:.6f}\n{eager}\n{fused}"
