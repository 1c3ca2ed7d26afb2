"""Drop-in encode / decode for the reference's residual vector quantisers on B200.

``MimiRVQB200`` mirrors ``MimiResidualVectorQuantizer`` (src/fast_mimi/model.py:2365-2444): ``encode(embeddings
[B, hidden, T], num_quantizers) -> int64 [K, B, T]`` and ``decode(codes [B, K, T]) -> float32 [B, hidden, T]``;
``MimiSplitRVQB200`` mirrors ``MimiSplitResidualVectorQuantizer`` (src/fast_mimi/model.py:2447-2480): one semantic
stack plus one acoustic stack on the same embeddings.  The 1 x 1 convolutions ``input_proj`` / ``output_proj`` run on
the tensor core as split-precision products (``ops.linear_split``: FP16 hi + lo parts, FP32 accumulation, the accuracy
of an FP32 linear, which the code decisions downstream need), the codebook search on ``ops.rvq_encode`` (tensor-core pre-selection, exact FP32 decision) and the
ordered sum on ``ops.rvq_decode``.  Codebook vectors are taken from the reference modules
(``layer.codebook.embed``) when the wrapper is built; rebuild it after loading new weights.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops


class MimiRVQB200:
    def __init__(self, codebooks: torch.Tensor, input_proj: torch.Tensor | None, output_proj: torch.Tensor | None) -> None:
        self.books = ops.RVQCodebooks(codebooks)
        flat = lambda w: None if w is None else w.detach().float().reshape(w.shape[0], -1).contiguous()
        self.input_proj, self.output_proj = flat(input_proj), flat(output_proj)
        # FP16 hi + lo parts of the projection weights for the tensor-core products
        self._in_parts = None if self.input_proj is None else ops.split_half(self.input_proj)
        self._out_parts = None if self.output_proj is None else ops.split_half(self.output_proj)

    @staticmethod
    def _project(x: torch.Tensor, w: torch.Tensor, parts) -> torch.Tensor:
        # the tensor-core kernel takes K in multiples of 64 and N in multiples of 256 (Mimi: 512 -> 256 and back);
        # other geometries (the reference's tiny test configuration) take the FP32 CUDA-core kernel
        if w.shape[1] % 64 == 0 and w.shape[0] % 256 == 0:
            return ops.linear_split(x, parts)
        return ops.linear_fp32(x, w)

    @classmethod
    def from_reference(cls, rvq: nn.Module) -> "MimiRVQB200":
        """``rvq``: a module with the reference's attributes ``layers[i].codebook.embed``, ``input_proj``,
        ``output_proj`` (1 x 1 ``nn.Conv1d`` without bias, or ``None``)."""
        books = torch.stack([layer.codebook.embed.detach().float() for layer in rvq.layers])
        weight = lambda conv: None if conv is None else conv.weight
        return cls(books, weight(rvq.input_proj), weight(rvq.output_proj))

    def encode(self, embeddings: torch.Tensor, num_quantizers: int | None = None) -> torch.Tensor:
        ops._need(embeddings.is_cuda and embeddings.dim() == 3, "embeddings must be CUDA [batch, channels, frames]")
        B, _, T = embeddings.shape
        x = embeddings.float().permute(0, 2, 1).reshape(B * T, -1)
        if self.input_proj is not None:
            x = self._project(x.contiguous(), self.input_proj, self._in_parts)
        codes = ops.rvq_encode(x.contiguous(), self.books, num_quantizers)
        # codes are the end of the device pipeline: a recorded error (a timed-out wait in a kernel upstream, a
        # non-finite residual) must not leave as plausible-looking indices
        ops.check_status(embeddings.device)
        return codes.view(codes.shape[0], B, T)

    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        ops._need(codes.is_cuda and codes.dim() == 3, "codes must be CUDA [batch, quantizers, frames]")
        B, K, T = codes.shape
        q = ops.rvq_decode(codes.transpose(0, 1).reshape(K, B * T).contiguous(), self.books)
        if self.output_proj is not None:
            q = self._project(q, self.output_proj, self._out_parts)
        return q.view(B, T, -1).permute(0, 2, 1).contiguous()


class MimiSplitRVQB200:
    def __init__(self, semantic: MimiRVQB200, acoustic: MimiRVQB200) -> None:
        self.semantic, self.acoustic = semantic, acoustic
        self.num_semantic_quantizers = semantic.books.layers
        self.max_num_quantizers = semantic.books.layers + acoustic.books.layers

    @classmethod
    def from_reference(cls, split: nn.Module) -> "MimiSplitRVQB200":
        return cls(MimiRVQB200.from_reference(split.semantic_residual_vector_quantizer),
                   MimiRVQB200.from_reference(split.acoustic_residual_vector_quantizer))

    def encode(self, embeddings: torch.Tensor, num_quantizers: int | None = None) -> torch.Tensor:
        count = self.max_num_quantizers if num_quantizers is None else int(num_quantizers)
        if not self.num_semantic_quantizers <= count <= self.max_num_quantizers:
            raise ValueError(f"num_quantizers must be in [{self.num_semantic_quantizers}, {self.max_num_quantizers}]")
        codes = self.semantic.encode(embeddings)
        if count > self.num_semantic_quantizers:
            codes = torch.cat((codes, self.acoustic.encode(embeddings, count - self.num_semantic_quantizers)), dim=0)
        return codes

    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        """``codes [B, K, T]``: semantic layers first (src/fast_mimi/model.py:2408-2444 per branch); the two
        branches' outputs are added."""
        n_sem = self.num_semantic_quantizers
        out = self.semantic.decode(codes[:, :n_sem].contiguous())
        if codes.shape[1] > n_sem:
            out = out + self.acoustic.decode(codes[:, n_sem:].contiguous())
        return out
