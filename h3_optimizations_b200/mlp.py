"""Chunked FP8-E4M3 MLP of the DiT block on the tcgen05 tensor cores.

The step behind the attention in a block: ``fc1`` (hidden -> ffn), GELU with
the tanh approximation, ``fc2`` (ffn -> hidden), executed in 4096-token chunks
so that the ``(tokens, ffn)`` intermediate never exists for the whole sequence.
Takes the place of the reference's bounded-memory MLP execution
(memory/forward.py:138-298 with the FP8 linears of memory/linear.py:352-492;
the reference model's MLP is a SwiGLU, the benchmark configuration this follows
specifies GELU-tanh 3072 -> 12288 -> 3072).

Formats: weights are quantised once, per output row, to E4M3 with
``scale = max(amax/448, 1e-20)``; activations are quantised per token the same
way in front of each GEMM (``h3s_quant_rows_fp8``).  Each GEMM is
``h3s_dense_gemm`` with E4M3 operands, FP32 accumulation and the two scales,
the bias and (for ``fc1``) the activation applied in its epilogue.
"""

from __future__ import annotations

import torch

from . import ops

CHUNK_ROWS = 4096
FP8_MAX = 448.0


def quantize_weight_rows_fp8(weight):
    """``(codes e4m3 (out, in), scale fp32 (out,))`` of a Linear weight, one
    scale per output row.  One-time preparation; runs wherever the weight lives."""
    w = weight.detach().float()
    scale = (w.abs().amax(dim=1) / FP8_MAX).clamp_min(1.0e-20)
    codes = (w / scale[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return codes.contiguous(), scale.contiguous()


class ChunkedFP8MLP:
    name = "chunked_b200_fp8_mlp"

    def __init__(self, fc1_weight, fc1_bias, fc2_weight, fc2_bias, *, chunk_rows=CHUNK_ROWS):
        if fc1_weight.ndim != 2 or fc2_weight.ndim != 2 or fc2_weight.shape[1] != fc1_weight.shape[0]:
            raise ValueError("fc1 (ffn, hidden) and fc2 (hidden_out, ffn) shapes do not chain")
        if int(chunk_rows) <= 0 or int(chunk_rows) % 128:
            raise ValueError("chunk_rows must be a positive multiple of 128")
        self.chunk_rows = int(chunk_rows)
        self.hidden, self.ffn, self.out_features = fc1_weight.shape[1], fc1_weight.shape[0], fc2_weight.shape[0]
        if self.hidden % 128 or self.ffn % 128 or self.out_features % 8:
            raise ValueError("hidden and ffn must be multiples of 128, the output width a multiple of 8")
        self.w1, self.w1_scale = quantize_weight_rows_fp8(fc1_weight)
        self.w2, self.w2_scale = quantize_weight_rows_fp8(fc2_weight)
        self.b1 = None if fc1_bias is None else fc1_bias.detach().float().contiguous()
        self.b2 = None if fc2_bias is None else fc2_bias.detach().float().contiguous()

    def to(self, device):
        for name in ("w1", "w1_scale", "w2", "w2_scale", "b1", "b2"):
            value = getattr(self, name)
            if value is not None:
                setattr(self, name, value.to(device))
        return self

    def __call__(self, x, out=None):
        """``x``: (tokens, hidden) bf16 on the GPU -> (tokens, out_features) bf16."""
        if x.ndim != 2 or x.dtype != torch.bfloat16 or not x.is_cuda or x.shape[1] != self.hidden:
            raise ValueError("x must be a CUDA bf16 tensor of shape (tokens, %d)" % self.hidden)
        tokens = x.shape[0]
        if out is None:
            out = torch.empty((tokens, self.out_features), dtype=torch.bfloat16, device=x.device)
        rows = min(self.chunk_rows, tokens)
        # chunk-sized scratch, reused by every chunk: the (tokens, ffn) intermediate is never whole
        x8 = torch.empty((rows, self.hidden), dtype=torch.float8_e4m3fn, device=x.device)
        h = torch.empty((rows, self.ffn), dtype=torch.bfloat16, device=x.device)
        h8 = torch.empty((rows, self.ffn), dtype=torch.float8_e4m3fn, device=x.device)
        x_scale = torch.empty((rows,), dtype=torch.float32, device=x.device)
        h_scale = torch.empty((rows,), dtype=torch.float32, device=x.device)
        for start in range(0, tokens, self.chunk_rows):
            stop = min(start + self.chunk_rows, tokens)
            n = stop - start
            ops.quant_rows_fp8(x[start:stop], x8, x_scale)
            ops.dense_gemm(x8[:n], self.w1, row_scale=x_scale[:n], col_scale=self.w1_scale, bias=self.b1,
                           activation="gelu_tanh", out=h[:n])
            ops.quant_rows_fp8(h[:n], h8, h_scale)
            ops.dense_gemm(h8[:n], self.w2, row_scale=h_scale[:n], col_scale=self.w2_scale, bias=self.b2,
                           out=out[start:stop])
        return out
