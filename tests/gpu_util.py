"""Helpers shared by the GPU parity tests."""
import torch

DEV = "cuda"


def to_dev(d):
    return {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in d.items()}


def bits(t: torch.Tensor) -> torch.Tensor:
    """Bit pattern view for exact comparison of 16-bit floats."""
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16)
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    return t


class Canary:
    """Allocates a tensor inside a larger buffer filled with a sentinel and checks, afterwards, that nothing
    outside the tensor was written (stands in for a memory checker)."""

    def __init__(self, shape, dtype, fill=0, pad=256):
        n = 1
        for s in shape:
            n *= s
        self.pad = pad
        self.buf = torch.empty(n + 2 * pad, dtype=dtype, device=DEV)
        self.sentinel = 0x5A if dtype in (torch.int8, torch.uint8) else 12345
        self.buf.fill_(self.sentinel)
        self.t = self.buf[pad:pad + n].view(shape)
        self.t.fill_(fill)

    def check(self, what=""):
        lo = self.buf[:self.pad]
        hi = self.buf[self.pad + self.t.numel():]
        assert bool((lo == self.sentinel).all()) and bool((hi == self.sentinel).all()), f"{what}: write outside the buffer"


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream
