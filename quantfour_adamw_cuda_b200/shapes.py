"""Parameter-shape lists of the benchmark workloads (tensor shapes only: no weights, no data)."""
from __future__ import annotations

import math
from typing import List, Tuple

Shape = Tuple[int, ...]


def llama(layers: int, hidden: int, mlp: int, vocab: int) -> List[Shape]:
    """Decoder stack: per layer 4 attention matrices, 3 MLP matrices, 2 norm vectors; plus the
    embedding and the LM head."""
    out: List[Shape] = [(vocab, hidden)]
    for _ in range(layers):
        out += [(hidden, hidden)] * 4 + [(mlp, hidden)] * 2 + [(hidden, mlp)] + [(hidden,)] * 2
    out.append((vocab, hidden))
    return out


def llama_7b() -> List[Shape]:
    return llama(32, 4096, 11008, 32000)


def llama_13b() -> List[Shape]:
    return llama(40, 5120, 13824, 32000)


def gpt2_medium() -> List[Shape]:
    """24 layers, hidden 1024: fused QKV, attention output, 4x MLP pair, biases, two LayerNorms per
    layer; token and position embeddings; final LayerNorm (about 355 M parameters)."""
    h = 1024
    out: List[Shape] = [(50257, h), (1024, h)]
    for _ in range(24):
        out += [(h,), (h,), (3 * h, h), (3 * h,), (h, h), (h,), (h,), (h,), (4 * h, h), (4 * h,), (h, 4 * h), (h,)]
    out += [(h,), (h,)]
    return out


WORKLOADS = {"llama7b": llama_7b, "llama13b": llama_13b, "gpt2m": gpt2_medium}


def numel(shapes: List[Shape]) -> int:
    return sum(math.prod(s) for s in shapes)


def algorithmic_bytes(shapes: List[Shape], elem_bytes: int = 2, threshold: int = 4096) -> int:
    """Compulsory HBM bytes of one step: parameter read + write, gradient read, both code buffers
    read + write, every scale read + written once; fp32-state tensors: parameter r/w, gradient, and
    both fp32 moments r/w."""
    total = 0
    for s in shapes:
        n = math.prod(s)
        if n <= threshold:
            total += n * (3 * elem_bytes + 16)
            continue
        nblk = (n + 127) // 128
        total += n * 3 * elem_bytes + 4 * ((n + 1) // 2) + 8 * nblk
        total += 8 * (s[0] + s[1]) if len(s) == 2 else 8 * nblk
    return total
