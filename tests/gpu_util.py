"""Helpers shared by the GPU parity tests: host <-> device moves and guarded outputs."""
import numpy as np
import torch

CANARY = 0x5A


def dev(a: np.ndarray) -> torch.Tensor:
    """numpy -> CUDA tensor with the same bytes (uint32/uint16/float16 go through int views)."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda()
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    if a.dtype == np.float16:
        return torch.from_numpy(a.view(np.int16)).cuda().view(torch.float16)
    return torch.from_numpy(a).cuda()


def host(t: torch.Tensor, dtype=None) -> np.ndarray:
    torch.cuda.synchronize()
    if t.dtype == torch.float16:
        a = t.view(torch.int16).cpu().numpy().view(np.float16)
    else:
        a = t.cpu().numpy()
    return a if dtype is None else a.view(dtype)


class Guarded:
    """A device output buffer with 256 canary bytes on either side."""

    def __init__(self, nbytes: int, align_offset: int = 0):
        self.n = nbytes
        self.off = 256 + align_offset
        self.raw = torch.full((nbytes + 512 + align_offset,), CANARY, dtype=torch.uint8, device="cuda")

    @property
    def ptr(self) -> int:
        return self.raw.data_ptr() + self.off

    def read(self, dtype) -> np.ndarray:
        torch.cuda.synchronize()
        raw = self.raw.cpu().numpy()
        assert (raw[: self.off] == CANARY).all(), "write before the output buffer"
        assert (raw[self.off + self.n:] == CANARY).all(), "write past the output buffer"
        return raw[self.off: self.off + self.n].copy().view(dtype)
