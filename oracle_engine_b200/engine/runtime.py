"""What every part is built with: the compute precision and the device.

`dtype` is the type of activations, matrix weights and the cache: bfloat16 (serving; the
tensor-core kernels) or float32 (the true 32-bit path: CUDA-core products, no reduced-
precision mode anywhere).  The residual stream, norms, softmax, rotary tables and logits
are float32 in both.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}") from None


@dataclass
class Runtime:
    dtype: torch.dtype
    device: torch.device
    tensor_cores: bool = True          # bf16 only: use the tcgen05 / mma kernels where they take the shape
    # A hint for the part that runs now: the weight matrix that the part after it streams first (or
    # None).  The model and the block set it before they call a part; a part's last product may ask
    # the first megabytes of it into the L2 while its own epilogue runs (csrc/ops_tc.py: gemm(then=)).
    next_weights: torch.Tensor | None = None
    # The float32 residual stream rounded to bfloat16, left by the kernel that last added into it (a norm's
    # add_into(..., keep_cast=True)): (address of the stream, the copy).  `activations` takes it instead of casting
    # again; the model clears it when a forward pass starts.
    cast_cache: tuple | None = None
    # Tensors that parts of different layers share during ONE forward pass (a history of the stream, say): the part
    # that runs first puts them here, the others find them.  While a CUDA graph is captured they are the graph's memory.
    pass_store: dict = field(default_factory=dict, repr=False)
    _buffers: dict = field(default_factory=dict, repr=False)
    _cast_turn: int = 0

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    def buffer(self, tag: str, *shape, dtype=None) -> torch.Tensor:
        """A tensor for an intermediate result of a step, kept under `tag` and handed out again at the next
        request for that tag (whatever the shape: the storage grows to the largest one asked for).  A prompt
        step of thousands of tokens asks for dozens of buffers of tens of megabytes in every layer; kept
        buffers take those requests away from the caching allocator.  Two results that are alive at the same time
        need different tags; everything runs on one stream, so a buffer's next user writes after its last
        reader has run.  While a CUDA graph is being captured this is `empty` (the graph owns its memory)."""
        dtype = dtype or self.dtype
        if self.device.type != "cuda" or torch.cuda.is_current_stream_capturing():
            return self.empty(*shape, dtype=dtype)
        n = 1
        for d in shape:
            n *= int(d)
        key = (tag, dtype)
        flat = self._buffers.get(key)
        if flat is None or flat.numel() < n:
            flat = None
            self._buffers.pop(key, None)
            flat = torch.empty(max(n + n // 4, 1), dtype=dtype, device=self.device)
            self._buffers[key] = flat
        return flat[:n].view(*shape)

    def activations(self, x: torch.Tensor) -> torch.Tensor:
        """The float32 residual stream as a sublayer's input: itself on the 32-bit path (the sublayer
        must not write to it), rounded to bfloat16 otherwise."""
        if self.dtype == torch.float32:
            return x
        cached, self.cast_cache = self.cast_cache, None
        if cached is not None and cached[0] == x.data_ptr() and cached[1].shape == x.shape:
            return cached[1]
        from ..csrc import ops
        y = self.buffer("activations", *x.shape)
        ops.cast_rows(y, x)
        return y

    def to_compute(self, t: torch.Tensor) -> torch.Tensor:
        """A stored matrix in the compute dtype (bf16 -> float32 is exact; a 32-bit
        matrix is rounded to bf16 only for the bf16 path)."""
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def to_f32(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=torch.float32).contiguous()
