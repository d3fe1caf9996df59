"""The operators inside their real caller: one decode step of a gpt-fast style Llama transformer block (RMSNorm,
rotary attention with a KV cache, SwiGLU feed-forward; the block of torchao/_models/llama/model.py) on random weights,
quantized with quantize(model, int4_weight_only(...)) and compiled the way the reference's generate.py compiles
decode_one_token (torchao/_models/llama/generate.py:222-228): torch.compile(mode="reduce-overhead", fullgraph=True).
The compiled step must contain the dispatcher operators (torch.ops.torchao._weight_int4pack_mm), replay under CUDA
graphs, and agree with eager execution within 1e-2.  Tokens per second and model_size * tokens/s are printed as
generate.py:292-305 prints them (run with -s to see them)."""
import time

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


class RMSNorm(torch.nn.Module):
    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(dim))

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x) * self.weight


def rotate(x, freqs):
    """x [B, S, H, D], freqs [S, D/2, 2] (cos, sin)."""
    xs = x.float().reshape(*x.shape[:-1], -1, 2)
    f = freqs.view(1, xs.size(1), 1, xs.size(3), 2)
    out = torch.stack([xs[..., 0] * f[..., 0] - xs[..., 1] * f[..., 1], xs[..., 1] * f[..., 0] + xs[..., 0] * f[..., 1]], -1)
    return out.flatten(3).type_as(x)


class Block(torch.nn.Module):
    """Pre-norm attention + feed-forward block with a static KV cache (one sequence, decode of one token at a time)."""

    def __init__(self, dim=4096, n_heads=32, n_kv_heads=8, hidden=14336, max_seq=256, dtype=torch.bfloat16):
        super().__init__()
        self.n_heads, self.n_kv, self.head_dim, self.dim = n_heads, n_kv_heads, dim // n_heads, dim
        self.wqkv = torch.nn.Linear(dim, (n_heads + 2 * n_kv_heads) * self.head_dim, bias=False)
        self.wo = torch.nn.Linear(dim, dim, bias=False)
        self.w1 = torch.nn.Linear(dim, hidden, bias=False)
        self.w3 = torch.nn.Linear(dim, hidden, bias=False)
        self.w2 = torch.nn.Linear(hidden, dim, bias=False)
        self.attention_norm, self.ffn_norm = RMSNorm(dim), RMSNorm(dim)
        self.register_buffer("k_cache", torch.zeros(1, n_kv_heads, max_seq, self.head_dim, dtype=dtype), persistent=False)
        self.register_buffer("v_cache", torch.zeros(1, n_kv_heads, max_seq, self.head_dim, dtype=dtype), persistent=False)
        pos = torch.arange(max_seq).float()
        inv = 1.0 / (500000.0 ** (torch.arange(0, self.head_dim, 2).float() / self.head_dim))
        ang = torch.outer(pos, inv)
        self.register_buffer("freqs", torch.stack([ang.cos(), ang.sin()], -1), persistent=False)
        self.register_buffer("mask", torch.tril(torch.ones(max_seq, max_seq, dtype=torch.bool)), persistent=False)

    def forward(self, x, input_pos):
        """x [1, S, dim], input_pos [S] (positions of these tokens)."""
        B, S, _ = x.shape
        h = self.attention_norm(x)
        q, k, v = self.wqkv(h).split([self.n_heads * self.head_dim, self.n_kv * self.head_dim, self.n_kv * self.head_dim], -1)
        q = rotate(q.view(B, S, self.n_heads, self.head_dim), self.freqs[input_pos]).transpose(1, 2)
        k = rotate(k.view(B, S, self.n_kv, self.head_dim), self.freqs[input_pos]).transpose(1, 2)
        v = v.view(B, S, self.n_kv, self.head_dim).transpose(1, 2)
        self.k_cache[:, :, input_pos] = k
        self.v_cache[:, :, input_pos] = v
        rep = self.n_heads // self.n_kv
        keys, vals = self.k_cache.repeat_interleave(rep, 1), self.v_cache.repeat_interleave(rep, 1)
        att = F.scaled_dot_product_attention(q, keys, vals, attn_mask=self.mask[None, None, input_pos])
        x = x + self.wo(att.transpose(1, 2).reshape(B, S, self.dim))
        h = self.ffn_norm(x)
        return x + self.w2(F.silu(self.w1(h)) * self.w3(h))


def _model_size_bytes(model):
    """Bytes of the parameters as stored (quantized weights count their packed tensors), generate.py:286 style."""
    total = 0
    for p in model.parameters():
        inner = getattr(p, "layout_tensor", None)
        if inner is not None:
            total += inner.packed_weight.numel() * inner.packed_weight.element_size()
            total += inner.scale_and_zero.numel() * inner.scale_and_zero.element_size()
        else:
            total += p.numel() * p.element_size()
    return total


def test_compiled_decode_step_of_a_llama_block():
    from torchao.quantization import int4_weight_only, quantize   # the reference's import names
    torch.manual_seed(0)
    dev = "cuda"
    with torch.device(dev):
        block = Block().to(torch.bfloat16).eval()
    for p in block.parameters():
        if p.dim() == 2:
            torch.nn.init.normal_(p, std=0.02)
    quantize(block, int4_weight_only(group_size=64))

    @torch.no_grad()
    def decode_one_token(x, input_pos):
        return block(x, input_pos)

    xs = [torch.randn(1, 1, 4096, device=dev, dtype=torch.bfloat16) for _ in range(8)]
    pos = [torch.tensor([i], device=dev, dtype=torch.int64) for i in range(8)]
    eager = [decode_one_token(x, p).clone() for x, p in zip(xs, pos)]
    block.k_cache.zero_()
    block.v_cache.zero_()
    compiled = torch.compile(decode_one_token, mode="reduce-overhead", fullgraph=True)
    outs = []
    for x, p in zip(xs, pos):
        outs.append(compiled(x, p).clone())
    for i, (a, b) in enumerate(zip(outs, eager)):
        err = float((a.float() - b.float()).abs().max() / b.float().abs().max())
        assert err <= 1e-2, f"token {i}: compiled and eager differ by {err}"

    # the graph the compiler backend receives (after the tensor subclasses have been traced through) holds the
    # dispatcher operator on the packed weight, not an opaque Python call
    from torch._dynamo.backends.common import aot_autograd
    seen = []

    def inspect(gm, example_inputs):
        seen.append(gm.print_readable(print_output=False))
        return gm.forward

    torch._dynamo.reset()
    probe = torch.compile(decode_one_token, backend=aot_autograd(fw_compiler=inspect), fullgraph=True)
    probe(xs[0], pos[0])
    assert any("torchao._weight_int4pack_mm" in g for g in seen), "the compiled graph does not contain the operator"

    # tokens per second of the block and model_size * tokens/s, as generate.py:292-305 reports them
    def rate(fn, n=200):
        for i in range(8):
            fn(xs[i % 8], pos[i % 8])
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(n):
            fn(xs[i % 8], pos[i % 8])
        torch.cuda.synchronize()
        return n / (time.perf_counter() - t0)

    torch._dynamo.reset()
    compiled = torch.compile(decode_one_token, mode="reduce-overhead", fullgraph=True)
    size = _model_size_bytes(block)
    for name, fn in (("eager", decode_one_token), ("compiled", compiled)):
        tps = rate(fn)
        print(f"[llama block, int4 g64, {name}] {tps:.1f} block-tokens/s, model size {size / 1e9:.3f} GB, "
              f"bandwidth achieved {size * tps / 1e9:.1f} GB/s")
