"""Token embedding (row gather into the float32 residual stream) and the output head (final hidden rows times the
head matrix, float32 logits). A tied head names the embedding's tensor and shares its device copy
(reference: src/etalii_dllm/transformer.py:659-663, 427-443)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .norm import project, row_rule
from .registry import register_part
from .spec import ParamSpec


class TokenEmbedding:
    def __init__(self, vocab_size: int, hidden_size: int) -> None:
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight = None

    @staticmethod
    def parameters(vocab_size, hidden_size) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((vocab_size, hidden_size))}

    def bind(self, tensors, rt) -> None:
        self.weight = rt.to_device(tensors["weight"], rt.dtype)

    def forward(self, tokens: torch.Tensor, n_tokens: int, rt) -> torch.Tensor:
        # a token outside the table sets the kernels' shared status word, which the engine looks at after each
        # step it waits for (kernels/ops.py::raise_if_failed)
        x = rt.ws.buffer("residual", (n_tokens, self.hidden_size), torch.float32)
        ops.embed(x, self.weight, tokens)
        return x


class LinearHead:
    accepts_pending_norm = True

    def __init__(self, vocab_size: int, hidden_size: int) -> None:
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight = None

    @staticmethod
    def parameters(vocab_size, hidden_size) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((vocab_size, hidden_size))}

    def bind(self, tensors, rt) -> None:
        self.weight = rt.to_device(tensors["weight"], rt.dtype)

    def supports(self, rt) -> str | None:
        return row_rule(rt, hidden_size=self.hidden_size)

    def choose_greedy(self, hidden, rt, out: torch.Tensor) -> bool:
        """The greedy choice without logits: out[r] = argmax of row r's logits (lowest index on ties), made inside
        the head product. Returns False, having done nothing, where that kernel does not take the step."""
        from .norm import NormedInput, fuses_norm

        rows = hidden.shape[0]
        if not ops.head_argmax_supported(rows, self.weight):
            return False
        scratch = rt.ws.buffer("head_candidates", (ops.head_argmax_scratch(rows, self.vocab_size),), torch.float32)
        if isinstance(hidden, NormedInput):
            if fuses_norm(self.weight):
                ops.head_argmax(out, hidden.x, self.weight, scratch, norm_weight=hidden.weight, eps=hidden.eps)
                return True
            hidden = hidden.tensor()
        ops.head_argmax(out, hidden, self.weight, scratch)
        return True

    def forward(self, hidden, rt) -> torch.Tensor:
        """hidden: final-normed rows, or the norm still pending (`NormedInput`)."""
        logits = rt.ws.buffer("logits", (hidden.shape[0], self.vocab_size), torch.float32)
        project(logits, hidden, self.weight, ops.EPI_STORE_F32)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear", LinearHead)
