"""Launch the in-tree sm_100a cubins on PyTorch tensors.

One :class:`Kernels` object per GPU binds the device's primary context (the one PyTorch uses), loads
each cubin on first use, and launches entries on PyTorch's current stream. There is no eager
fallback: on a machine with a GPU a missing cubin or entry is an error, never a silent PyTorch path.
"""
from __future__ import annotations

import struct
import threading
from pathlib import Path

import torch

from .. import _native

KDIR = Path(__file__).resolve().parent.parent / "kernels"

# CUtensorMapDataType codes
TM_U8, TM_U16, TM_U32, TM_I32, TM_U64, TM_I64, TM_F16, TM_F32, TM_F64, TM_BF16 = range(10)

_TM_OF = {
    torch.uint8: TM_U8, torch.int8: TM_U8, torch.int32: TM_I32, torch.int64: TM_I64,
    torch.float16: TM_F16, torch.float32: TM_F32, torch.bfloat16: TM_BF16,
}
if hasattr(torch, "float8_e4m3fn"):
    _TM_OF[torch.float8_e4m3fn] = TM_U8


def ptr(t: torch.Tensor | None) -> bytes:
    return struct.pack("<Q", 0 if t is None else t.data_ptr())


def i32(v: int) -> bytes:
    return struct.pack("<i", int(v))


def u32(v: int) -> bytes:
    return struct.pack("<I", int(v))


def i64(v: int) -> bytes:
    return struct.pack("<q", int(v))


def f32(v: float) -> bytes:
    return struct.pack("<f", float(v))


class Kernels:
    """Per-GPU kernel registry and launcher."""

    _instances: dict[int, "Kernels"] = {}
    _lock = threading.Lock()

    def __init__(self, gpu: int):
        if not _native.cuda_available():
            raise RuntimeError("kern_b200 kernels need a CUDA device; none is available here")
        self.gpu = gpu
        self.dev = _native.Device(gpu)
        self._modules: dict[str, object] = {}
        self._functions: dict[tuple[str, str], object] = {}
        self._tmaps: dict[tuple, bytes] = {}
        self.launches = 0  # count of kernel launches issued through this object
        self._err = None

    @classmethod
    def get(cls, device: torch.device | int | None = None) -> "Kernels":
        if device is None:
            gpu = torch.cuda.current_device()
        elif isinstance(device, int):
            gpu = device
        else:
            gpu = device.index if device.index is not None else torch.cuda.current_device()
        with cls._lock:
            k = cls._instances.get(gpu)
            if k is None:
                torch.cuda.init()
                with torch.cuda.device(gpu):
                    torch.zeros(1, device="cuda")  # make sure the primary context exists
                k = cls._instances[gpu] = Kernels(gpu)
            return k

    @property
    def sm_count(self) -> int:
        return self.dev.sm_count

    def err_word(self) -> torch.Tensor:
        """A device int32 that kernels set when a bounded wait ran out or a checked index failed."""
        if self._err is None:
            self._err = torch.zeros(1, dtype=torch.int32, device=f"cuda:{self.gpu}")
        return self._err

    def check_error(self) -> None:
        code = int(self.err_word().item())
        if code:
            self._err.zero_()
            raise RuntimeError(f"kern_b200 kernel reported device error code {code}")

    def function(self, module: str, entry: str):
        key = (module, entry)
        f = self._functions.get(key)
        if f is None:
            mod = self._modules.get(module)
            if mod is None:
                path = KDIR / (module + ".cubin")
                if not path.exists():
                    raise RuntimeError(f"built-in kernel module {path} is missing: run kern_b200._build")
                mod = self._modules[module] = self.dev.load_module(path.read_bytes())
            f = self._functions[key] = self.dev.function(mod, entry)
        return f

    def launch(self, module: str, entry: str, grid, block, params: list[bytes], shared_mem: int = 0,
               cluster=(1, 1, 1), pdl: bool = False, stream: int | None = None) -> None:
        f = self.function(module, entry)
        if stream is None:
            stream = torch.cuda.current_stream(self.gpu).cuda_stream
        g = tuple(grid) + (1,) * (3 - len(grid))
        b = tuple(block) + (1,) * (3 - len(block))
        self.dev.launch(f, list(g), list(b), shared_mem, stream, params, list(cluster), pdl)
        self.launches += 1

    def tensor_map_2d(self, t: torch.Tensor, box_rows: int, box_cols: int, swizzle: int = 128,
                      rows: int | None = None) -> bytes:
        """Tiled TMA descriptor over a row-major 2-D view ``t[rows, cols]`` (last stride 1)."""
        assert t.dim() == 2 and t.stride(1) == 1, "tensor map needs a row-major 2-D tensor"
        es = t.element_size()
        nrows = t.shape[0] if rows is None else rows
        key = (t.data_ptr(), nrows, t.shape[1], t.stride(0), es, box_rows, box_cols, swizzle)
        tm = self._tmaps.get(key)
        if tm is None:
            tm = self.dev.encode_tensor_map(
                t.data_ptr(), _TM_OF[t.dtype], [t.shape[1], nrows], [t.stride(0) * es],
                [box_cols, box_rows], swizzle, 256, False)
            if len(self._tmaps) > 4096:
                self._tmaps.clear()
            self._tmaps[key] = tm
        return tm
