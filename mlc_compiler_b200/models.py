"""Benchmark model definitions and their seeded synthetic inputs.

The schedules shipped under ``schedules/`` were captured from these modules, so
their state-dict keys are what a schedule's parameter table refers to.  The
architectures are the ones the benchmark configurations name:

* ``bert-base``: 12 post-LN encoder layers, hidden 768, 12 heads of 64, FFN 3072
  with exact (erf) GELU, LayerNorm eps 1e-12, vocabulary 30522, 512 learned
  positions, 2 token types, pooled ``tanh`` output -- the same graph shape as the
  reference's benchmark model (``mlc/bench/models.py:49-110``);
* ``gpt2-small``: 12 pre-LN decoder layers, hidden 768, 12 heads, causal additive
  mask taken from a ``[1, 1, 1024, 1024]`` buffer, FFN 3072, vocabulary 50257,
  1024 learned positions.  ``gelu="tanh", tied_head=True`` is GPT-2 proper (the
  configuration the benchmark names); ``gelu="erf", tied_head=False`` is the
  variant the reference itself ships (``mlc/bench/models.py:113-175``);
* ``encoder-block``: one post-LN BERT layer on activations, the fp32 plumbing
  configuration.

Weights are synthetic: every matrix and embedding ~ N(0, 0.02), LayerNorm gain 1
and bias 0, linear biases 0, drawn after ``torch.manual_seed(0)``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class EncoderDims:
    vocab: int = 30522
    positions: int = 512
    layers: int = 12
    heads: int = 12
    hidden: int = 768
    ffn: int = 3072
    eps: float = 1e-12


@dataclass
class DecoderDims:
    vocab: int = 50257
    positions: int = 1024
    layers: int = 12
    heads: int = 12
    hidden: int = 768
    eps: float = 1e-5
    gelu: str = "tanh"      # "tanh" | "erf"
    tied_head: bool = True


def _split_heads(x: torch.Tensor, heads: int) -> torch.Tensor:
    b, t, d = x.shape
    return x.view(b, t, heads, d // heads).transpose(1, 2)


def _merge_heads(x: torch.Tensor) -> torch.Tensor:
    b, h, t, dh = x.shape
    return x.transpose(1, 2).reshape(b, t, h * dh)


class EncoderLayer(nn.Module):
    """Post-LN: ``LN(x + sublayer(x))`` twice."""

    def __init__(self, d: EncoderDims):
        super().__init__()
        self.heads = d.heads
        self.scale = math.sqrt(d.hidden // d.heads)
        self.q = nn.Linear(d.hidden, d.hidden)
        self.k = nn.Linear(d.hidden, d.hidden)
        self.v = nn.Linear(d.hidden, d.hidden)
        self.o = nn.Linear(d.hidden, d.hidden)
        self.attn_norm = nn.LayerNorm(d.hidden, eps=d.eps)
        self.up = nn.Linear(d.hidden, d.ffn)
        self.down = nn.Linear(d.ffn, d.hidden)
        self.ffn_norm = nn.LayerNorm(d.hidden, eps=d.eps)

    def forward(self, x, mask):
        q = _split_heads(self.q(x), self.heads)
        k = _split_heads(self.k(x), self.heads)
        v = _split_heads(self.v(x), self.heads)
        probs = ((q @ k.transpose(-2, -1)) / self.scale + mask).softmax(dim=-1)
        x = self.attn_norm(x + self.o(_merge_heads(probs @ v)))
        return self.ffn_norm(x + self.down(F.gelu(self.up(x))))


class EncoderBlock(nn.Module):
    """One encoder layer on activations with an additive mask."""

    def __init__(self, d: EncoderDims = EncoderDims()):
        super().__init__()
        self.layer = EncoderLayer(d)

    def forward(self, x, mask):
        return self.layer(x, mask)


class BertEncoder(nn.Module):
    def __init__(self, d: EncoderDims = EncoderDims()):
        super().__init__()
        self.dims = d
        self.tok = nn.Embedding(d.vocab, d.hidden)
        self.pos = nn.Embedding(d.positions, d.hidden)
        self.typ = nn.Embedding(2, d.hidden)
        self.emb_norm = nn.LayerNorm(d.hidden, eps=d.eps)
        self.layers = nn.ModuleList(EncoderLayer(d) for _ in range(d.layers))
        self.pool = nn.Linear(d.hidden, d.hidden)
        self.register_buffer("position_ids", torch.arange(d.positions), persistent=False)

    def forward(self, input_ids, attention_mask):
        t = input_ids.shape[1]
        x = self.tok(input_ids) + self.pos(self.position_ids[:t]) + self.typ(
            torch.zeros_like(input_ids))
        x = self.emb_norm(x)
        mask = (1.0 - attention_mask[:, None, None, :]) * torch.finfo(torch.float32).min
        for layer in self.layers:
            x = layer(x, mask)
        return torch.tanh(self.pool(x[:, 0]))


class DecoderLayer(nn.Module):
    """Pre-LN: ``x + sublayer(LN(x))`` twice."""

    def __init__(self, d: DecoderDims):
        super().__init__()
        self.heads = d.heads
        self.scale = math.sqrt(d.hidden // d.heads)
        self.approx = "tanh" if d.gelu == "tanh" else "none"
        self.attn_norm = nn.LayerNorm(d.hidden, eps=d.eps)
        self.qkv = nn.Linear(d.hidden, 3 * d.hidden)
        self.o = nn.Linear(d.hidden, d.hidden)
        self.ffn_norm = nn.LayerNorm(d.hidden, eps=d.eps)
        self.up = nn.Linear(d.hidden, 4 * d.hidden)
        self.down = nn.Linear(4 * d.hidden, d.hidden)

    def forward(self, x, causal):
        t = x.shape[1]
        q, k, v = self.qkv(self.attn_norm(x)).chunk(3, dim=-1)
        q, k, v = (_split_heads(z, self.heads) for z in (q, k, v))
        scores = (q @ k.transpose(-2, -1)) / self.scale + causal[:, :, :t, :t]
        x = x + self.o(_merge_heads(scores.softmax(dim=-1) @ v))
        return x + self.down(F.gelu(self.up(self.ffn_norm(x)), approximate=self.approx))


class GPT2(nn.Module):
    def __init__(self, d: DecoderDims = DecoderDims()):
        super().__init__()
        self.dims = d
        self.tok = nn.Embedding(d.vocab, d.hidden)
        self.pos = nn.Embedding(d.positions, d.hidden)
        self.layers = nn.ModuleList(DecoderLayer(d) for _ in range(d.layers))
        self.final_norm = nn.LayerNorm(d.hidden, eps=d.eps)
        self.head = nn.Linear(d.hidden, d.vocab, bias=False)
        if d.tied_head:
            self.head.weight = self.tok.weight
        keep = torch.tril(torch.ones(d.positions, d.positions))
        self.register_buffer("causal", ((1.0 - keep) * torch.finfo(torch.float32).min)
                             .view(1, 1, d.positions, d.positions), persistent=False)
        self.register_buffer("position_ids", torch.arange(d.positions), persistent=False)

    def forward(self, input_ids):
        t = input_ids.shape[1]
        x = self.tok(input_ids) + self.pos(self.position_ids[:t])
        for layer in self.layers:
            x = layer(x, self.causal)
        return self.head(self.final_norm(x))


# --------------------------------------------------------------------------
# fused-kernel microbenchmark modules (one generated kernel each)
# --------------------------------------------------------------------------

class LayerNormRows(nn.Module):
    """LayerNorm over ``[rows, 768]``."""

    def __init__(self, hidden: int = 768, eps: float = 1e-5):
        super().__init__()
        self.norm = nn.LayerNorm(hidden, eps=eps)

    def forward(self, x):
        return self.norm(x)


class CausalSoftmax(nn.Module):
    """``softmax(x / 8 + causal_mask)`` over ``[B, 12, S, S]``."""

    def __init__(self, seq: int = 128):
        super().__init__()
        keep = torch.tril(torch.ones(seq, seq))
        self.register_buffer("mask", ((1.0 - keep) * torch.finfo(torch.float32).min)
                             .view(1, 1, seq, seq), persistent=False)

    def forward(self, x):
        return (x / 8.0 + self.mask).softmax(dim=-1)


class BiasGeluResidual(nn.Module):
    """``res + gelu(x + b)`` over ``[rows, 3072]``."""

    def __init__(self, width: int = 3072, approximate: str = "tanh"):
        super().__init__()
        self.bias = nn.Parameter(torch.zeros(width))
        self.approximate = approximate

    def forward(self, x, res):
        return res + F.gelu(x + self.bias, approximate=self.approximate)


# --------------------------------------------------------------------------

def init_weights(model: nn.Module, seed: int = 0, std: float = 0.02) -> nn.Module:
    """N(0, std) matrices and embeddings, unit LayerNorm, zero biases."""
    g = torch.Generator().manual_seed(seed)
    seen: set[int] = set()
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                if id(m.weight) not in seen:
                    seen.add(id(m.weight))
                    m.weight.copy_(torch.randn(m.weight.shape, generator=g) * std)
                if isinstance(m, nn.Linear) and m.bias is not None:
                    m.bias.zero_()
            elif isinstance(m, nn.LayerNorm):
                m.weight.fill_(1.0)
                m.bias.zero_()
    return model


def init_micro(model: nn.Module, seed: int = 0) -> nn.Module:
    """Microbenchmark parameters: gain 1 + N(0, 0.02), every bias N(0, 0.02)."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, nn.LayerNorm):
                m.weight.copy_(1.0 + torch.randn(m.weight.shape, generator=g) * 0.02)
                m.bias.copy_(torch.randn(m.bias.shape, generator=g) * 0.02)
            elif isinstance(m, BiasGeluResidual):
                m.bias.copy_(torch.randn(m.bias.shape, generator=g) * 0.02)
    return model


def _cast(model: nn.Module, args: tuple, dtype: torch.dtype):
    if dtype != torch.float32:
        model = model.to(dtype)
        args = tuple(a.to(dtype) if a.is_floating_point() else a for a in args)
    return model, args


def build(name: str, batch: int = 1, seq: int = 128, dtype: torch.dtype = torch.float32,
          seed: int = 0, **variant):
    """(model in eval mode, example inputs) for a named configuration, on CPU.
    Inputs are seeded: token ids uniform over the vocabulary, masks all ones,
    activations N(0, 1)."""
    g = torch.Generator().manual_seed(seed + 1)
    if name == "bert-base":
        d = EncoderDims(**variant)
        model = init_weights(BertEncoder(d), seed)
        args = (torch.randint(0, d.vocab, (batch, seq), generator=g), torch.ones(batch, seq))
    elif name == "gpt2-small":
        d = DecoderDims(**variant)
        model = init_weights(GPT2(d), seed)
        args = (torch.randint(0, d.vocab, (batch, seq), generator=g),)
    elif name == "encoder-block":
        d = EncoderDims(**variant)
        model = init_weights(EncoderBlock(d), seed)
        args = (torch.randn(batch, seq, d.hidden, generator=g), torch.zeros(batch, 1, 1, seq))
    elif name == "micro-layernorm":
        model = init_micro(LayerNormRows(**variant), seed)
        args = (torch.randn(batch * seq, model.norm.normalized_shape[0], generator=g),)
    elif name == "micro-softmax":
        model = CausalSoftmax(seq)
        args = (torch.randn(batch, 12, seq, seq, generator=g),)
    elif name == "micro-gelu":
        model = init_micro(BiasGeluResidual(**variant), seed)
        w = model.bias.shape[0]
        args = (torch.randn(batch * seq, w, generator=g), torch.randn(batch * seq, w, generator=g))
    else:
        raise KeyError(f"unknown model {name!r}")
    model = model.eval()
    return _cast(model, args, dtype)


def build_inputs(name: str, batch: int, seq: int = 128, dtype: torch.dtype = torch.float32,
                 seed: int = 0):
    """The seeded example inputs of ``build(name, batch, ...)`` without building the
    model (same generator, same draws) -- e.g. the whole batch that replicas split.
    Returns ``(None, inputs)`` so that it unpacks like :func:`build`."""
    g = torch.Generator().manual_seed(seed + 1)
    if name == "bert-base":
        args = (torch.randint(0, EncoderDims().vocab, (batch, seq), generator=g),
                torch.ones(batch, seq))
    elif name == "gpt2-small":
        args = (torch.randint(0, DecoderDims().vocab, (batch, seq), generator=g),)
    else:
        raise KeyError(f"no input recipe for {name!r}")
    if dtype != torch.float32:
        args = tuple(a.to(dtype) if a.is_floating_point() else a for a in args)
    return None, args


def schedule_name(name: str, batch: int, dtype: torch.dtype, seq: int = 128, tag: str = "") -> str:
    dt = str(dtype).replace("torch.", "")
    return f"{name}{('-' + tag) if tag else ''}_b{batch}_s{seq}_{dt}"
