"""GPT-2 (optimus_dl/modules/model/gpt2.py:34-338): learned positions, pre-LN blocks, GELU MLP,
tied embeddings, N(0, 0.02) init with scaled residual projections, decay / no-decay parameter
groups returned as named tuples, full-recompute sampling in ``generate``."""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import attention as attn_ops
from ..ops import embedding as emb_ops
from ..ops import linear as lin_ops
from . import register_model
from .base import BaseModel
from .blocks.attention import CausalSelfAttention
from .blocks.layer_norms import LayerNorm, RMSNorm
from .blocks.mlp import GELUMLP
from .config import ModelConfig

BLACKLIST_WEIGHT_MODULES = (nn.LayerNorm, LayerNorm, RMSNorm, nn.Embedding)


@dataclass
class GPTConfig(ModelConfig):
    block_size: int = 1024
    vocab_size: int = 50304
    n_layer: int = 12
    n_head: int = 12
    n_embd: int = 768
    head_dim: int | None = None
    dropout: float = 0.0
    bias: bool = True
    tie_word_embeddings: bool = True
    shard_every_ith_layer: int = 1
    padding_token_id: int | None = None


class MLP(GELUMLP):
    """GPT-2's feed-forward block under the name and with the constructor of the reference
    (optimus_dl/modules/model/gpt2.py:81-96): built from a config with ``n_embd``, ``bias`` and ``dropout``; the
    ``gelu`` and ``dropout`` sub-modules always exist."""

    def __init__(self, config):
        super().__init__(config.n_embd, 4 * config.n_embd, bias=config.bias, dropout=config.dropout)
        self.gelu = nn.GELU()
        if self.dropout is None:
            self.dropout = nn.Dropout(config.dropout)


class Block(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.ln_1 = LayerNorm(config.n_embd, bias=config.bias)
        self.attn = CausalSelfAttention(config)
        self.ln_2 = LayerNorm(config.n_embd, bias=config.bias)
        self.mlp = MLP(config)

    def forward(self, x, **kw):
        x = x + self.attn(self.ln_1(x), **kw)
        return x + self.mlp(self.ln_2(x))


@register_model("gpt2", GPTConfig)
class GPT(BaseModel):
    supports_fused_head = True

    def __init__(self, config, **_):
        super().__init__()
        assert config.vocab_size is not None and config.block_size is not None
        self.config = config
        self.transformer = nn.ModuleDict(self._build_transformer(config))
        self.lm_head = nn.Linear(config.n_embd, config.vocab_size, bias=False)
        if config.tie_word_embeddings:
            self.transformer.wte.weight = self.lm_head.weight
        self.apply(self._init_weights)
        self._init_residual_projections()

    def _build_transformer(self, config) -> dict:
        return dict(
            wte=nn.Embedding(config.vocab_size, config.n_embd, padding_idx=config.padding_token_id),
            wpe=nn.Embedding(config.block_size, config.n_embd),
            drop=nn.Dropout(config.dropout),
            h=nn.ModuleList([Block(config) for _ in range(config.n_layer)]),
            ln_f=LayerNorm(config.n_embd, bias=config.bias),
        )

    def _init_weights(self, module: nn.Module) -> None:
        if isinstance(module, nn.Linear):
            nn.init.normal_(module.weight, mean=0.0, std=0.02)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, mean=0.0, std=0.02)

    def _init_residual_projections(self) -> None:
        std = 0.02 / math.sqrt(2 * self.config.n_layer)
        for name, p in self.named_parameters():
            if name.endswith("c_proj.weight") or name.endswith("wo.weight"):
                nn.init.normal_(p, mean=0.0, std=std)

    # ------------------------------------------------------------------ forward
    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        if getattr(self, "_tp", None) is not None:
            from ..parallel import tp as tp_ops

            return tp_ops.embed_forward(self, input_ids)
        return emb_ops.embedding(input_ids, self.transformer.wte.weight, self.config.padding_token_id)

    def head(self, x: torch.Tensor) -> torch.Tensor:
        if getattr(self, "_tp", None) is not None:
            from ..parallel import tp as tp_ops

            return tp_ops.head_forward(self, x)
        return lin_ops.linear(x, self.lm_head.weight)

    def forward(self, input_ids: torch.Tensor, seq_lens=None, document_ids=None, position_ids=None, cu_seqlens=None,
                max_seqlen=None, skip_lm_head: bool = False, **kwargs):
        B, T = input_ids.shape
        assert T <= self.config.block_size, f"sequence of length {T} exceeds block size {self.config.block_size}"
        pos = position_ids if position_ids is not None else torch.arange(T, device=input_ids.device).unsqueeze(0)
        x = self.embed(input_ids) + F.embedding(pos, self.transformer.wpe.weight)
        x = self.transformer.drop(x)
        doc_start = attn_ops.build_doc_start(B, T, x.device, document_ids, cu_seqlens)
        for block in self.transformer.h:
            x = block(x, seq_lens=seq_lens, document_ids=document_ids, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen,
                      doc_start=doc_start)
        x = self.transformer.ln_f(x)
        if skip_lm_head:
            return {"hidden": x}
        return {"logits": self.head(x)}

    # ------------------------------------------------------------------ optimizer groups
    def is_decay_param(self, module: nn.Module, param_name: str) -> bool | None:
        if param_name.endswith("weight_clip_val") or param_name.endswith("bias"):
            return False
        if param_name.endswith("weight") and isinstance(module, nn.Linear):
            return True
        if param_name.endswith("weight") and isinstance(module, BLACKLIST_WEIGHT_MODULES):
            return False
        if param_name.endswith("gate_up_proj") or param_name.endswith("down_proj"):
            return True
        return None

    def make_parameter_groups(self):
        decay, no_decay = set(), set()
        for mn, m in self.named_modules():
            for pn, _ in m.named_parameters(recurse=False):
                fpn = f"{mn}.{pn}" if mn else pn
                d = self.is_decay_param(m, pn)
                if d is None:
                    continue
                (decay if d else no_decay).add(fpn)
        decay.discard("lm_head.weight")
        if self.lm_head.weight is not self.transformer.wte.weight:
            no_decay.add("lm_head.weight")
        names = {n for n, _ in self.named_parameters()}
        both = decay & no_decay
        assert not both, f"parameters {both} made it into both decay/no_decay sets!"
        missing = names - (decay | no_decay)
        assert not missing, f"parameters {missing} were not separated into either decay/no_decay set!"
        return [
            {"params": [(n, p) for n, p in self.named_parameters() if n in decay]},
            {"params": [(n, p) for n, p in self.named_parameters() if n in no_decay], "weight_decay": 0.0},
        ]

    # ------------------------------------------------------------------ sampling / sharding
    @torch.no_grad()
    def generate(self, idx: torch.Tensor, max_new_tokens: int, temperature: float = 1.0, top_k: int | None = None):
        limit = getattr(self.config, "block_size", None) or getattr(self.config, "sequence_length")
        for _ in range(max_new_tokens):
            cond = idx if idx.size(1) <= limit else idx[:, -limit:]
            logits = self(cond)["logits"][:, -1, :].float() / temperature
            if top_k is not None:
                v, _ = torch.topk(logits, min(top_k, logits.size(-1)))
                logits[logits < v[:, [-1]]] = -float("inf")
            nxt = torch.multinomial(F.softmax(logits, dim=-1), num_samples=1)
            idx = torch.cat((idx, nxt), dim=1)
        return idx

    def fully_shard(self, **fsdp_kwargs):
        """One sharding group per transformer block (the root group holds embeddings, final norm, head)."""
        return list(self.transformer.h)


@GPT.register_arch("124m")
def gpt2_124m():
    return GPTConfig(n_layer=12, n_head=12, n_embd=768)
