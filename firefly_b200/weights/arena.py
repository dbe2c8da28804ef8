"""One device arena for all of a model's weights, filled straight from their source.

The reference sizes one device chunk in a first pass over the checkpoint and bump-allocates
every tensor in it at 256-byte alignment (include/firefly/model_loader.h:48-58,
include/firefly/mm/model_weight_pool.h:58-109: ``ModelWeightPool``), reading from a mapping of
the file that is registered with the driver (include/firefly/mm/memory_mapper.h:117-135).  The
same here, with two additions.  Parts may ask for *fused* tensors (q|k|v stacked, gate and up
interleaved): the arena then holds only the fused matrix and each source tensor is copied
straight into its rows of it, so no matrix exists twice, not even for a moment.  And the source
need not be a file: seeded random weights are drawn into the same places by a kernel.

    plan   = ArenaPlan(weight_specs, fused_specs, device_dtype_of_each_source)
    arena  = WeightArena(plan, device)                   # the one allocation
    source.fill(arena)                                   # FileSource or RandomSource
    tensors = arena.tensors()                            # name -> view, for ``bind``

Copies run on a stream of their own; ``fill`` returns when they are done.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch

ALIGN = 256                      # bytes; the reference's alignment, and enough for TMA descriptors
STAGING_BYTES = 256 << 20        # device buffer that tensors of another stored type pass through

_WT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.float64: 3}


@dataclass(frozen=True)
class Piece:
    """Where one source tensor's rows go inside a fused tensor: source row r lands on row
    ``row0 + (r // group) * group_stride + r % group``; ``group`` 0 means one block of rows."""

    source: str
    row0: int
    group: int = 0
    group_stride: int = 0


@dataclass(frozen=True)
class FusedSpec:
    """A tensor of the arena that is put together from several source tensors (same trailing
    sizes, rows placed by ``pieces``).  The sources get no place of their own."""

    name: str
    shape: Tuple[int, ...]
    pieces: Tuple[Piece, ...]


@dataclass(frozen=True)
class Slot:
    name: str
    offset: int
    shape: Tuple[int, ...]
    dtype: torch.dtype

    @property
    def nbytes(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n * torch.empty((), dtype=self.dtype).element_size()


@dataclass(frozen=True)
class Placement:
    """One source tensor's destination: a slot and the placement of its rows in it."""

    slot: str
    row0: int
    group: int
    group_stride: int


def _rows_cols(shape: Sequence[int]) -> Tuple[int, int]:
    if len(shape) == 0:
        return 1, 1
    if len(shape) == 1:
        return 1, int(shape[0])
    cols = 1
    for s in shape[1:]:
        cols *= int(s)
    return int(shape[0]), cols


class ArenaPlan:
    """The first pass: which tensors the arena holds, where, and where each source goes."""

    def __init__(self, sources: Mapping[str, Tuple[Tuple[int, ...], torch.dtype]],
                 fused: Iterable[FusedSpec] = ()):
        """``sources``: name -> (shape, element type *on the device*) of every source tensor that is
        to be loaded.  ``fused``: tensors put together from some of them."""
        self.slots: Dict[str, Slot] = {}
        self.placements: Dict[str, Placement] = {}
        self.source_shapes = {n: tuple(s) for n, (s, _) in sources.items()}
        offset = 0

        def add(name, shape, dtype):
            nonlocal offset
            if name in self.slots:
                raise ValueError(f"arena tensor '{name}' is planned twice")
            slot = Slot(name, offset, tuple(int(s) for s in shape), dtype)
            self.slots[name] = slot
            offset += -(-slot.nbytes // ALIGN) * ALIGN
        for f in fused:
            dtypes = set()
            for p in f.pieces:
                if p.source not in sources:
                    raise KeyError(f"fused tensor '{f.name}' needs source '{p.source}', which is not loaded")
                shape, dt = sources[p.source]
                if tuple(shape[1:]) != tuple(f.shape[1:]):
                    raise ValueError(f"'{p.source}' {list(shape)} does not fit rows of '{f.name}' {list(f.shape)}")
                dtypes.add(dt)
            dtype = dtypes.pop() if len(dtypes) == 1 else torch.float32     # mixed sources: the wider type
            add(f.name, f.shape, dtype)
            for p in f.pieces:
                if p.source in self.placements:
                    raise ValueError(f"source '{p.source}' is placed twice")
                rows = int(sources[p.source][0][0])
                group = p.group or rows
                if rows % group:
                    raise ValueError(f"'{p.source}': {rows} rows are no multiple of the group of {group}")
                self.placements[p.source] = Placement(f.name, p.row0, group, p.group_stride or group)
        for name, (shape, dt) in sources.items():
            if name not in self.placements:
                add(name, shape, dt)
                rows, _ = _rows_cols(shape)
                self.placements[name] = Placement(name, 0, max(rows, 1), max(rows, 1))
        self.total_bytes = offset

    def check(self) -> None:
        """Every slot aligned, inside the arena, and overlapping no other."""
        end = 0
        for s in sorted(self.slots.values(), key=lambda s: s.offset):
            if s.offset % ALIGN or s.offset < end or s.offset + s.nbytes > self.total_bytes:
                raise AssertionError(f"arena slot '{s.name}' is misplaced")
            end = s.offset + s.nbytes


class WeightArena:
    """The one device allocation, and typed views of its slots."""

    def __init__(self, plan: ArenaPlan, device):
        self.plan = plan
        self.device = torch.device(device)
        self.buffer = torch.empty(max(plan.total_bytes, ALIGN), dtype=torch.uint8, device=self.device)
        if self.buffer.data_ptr() % ALIGN:
            raise RuntimeError("the device allocator returned an address that is not 256-byte aligned")

    def view(self, name: str) -> torch.Tensor:
        s = self.plan.slots[name]
        return self.buffer[s.offset: s.offset + s.nbytes].view(s.dtype).view(s.shape)

    def tensors(self) -> Dict[str, torch.Tensor]:
        return {n: self.view(n) for n in self.plan.slots}

    def destination(self, source: str) -> Tuple[torch.Tensor, Placement]:
        pl = self.plan.placements[source]
        return self.view(pl.slot), pl


# ----------------------------------------------------------------------------------------------
def _lib() -> ctypes.CDLL:
    from ..ops.build import load_module
    lib = load_module("weights.cu")
    lib.ff_weights_map_file.restype = c_void_p
    return lib


class MappedFile:
    """A checkpoint file mapped read-only and, where the driver allows, registered as pinned
    host memory so that copies from it are asynchronous (the reference's ``PinnedMappedFile`` idea,
    include/firefly/mm/memory_mapper.h:117-135).  A refused registration is not an error."""

    def __init__(self, path: str, register: bool = True):
        self.path = path
        addr, size, pinned, err = c_void_p(), c_ulonglong(), c_int(), c_int()
        self._lib = _lib()
        self._handle = self._lib.ff_weights_map_file(os.fsencode(path), c_int(1 if register else 0),
                                                    ctypes.byref(addr), ctypes.byref(size), ctypes.byref(pinned),
                                                    ctypes.byref(err))
        if not self._handle:
            raise OSError(err.value, f"cannot map '{path}': {os.strerror(err.value)}")
        self.address = addr.value or 0
        self.size = size.value
        self.pinned = pinned.value == 1
        self.refusal = -pinned.value if pinned.value < 0 else 0     # the driver's error code when it would not pin

    def close(self) -> None:
        if self._handle:
            self._lib.ff_weights_unmap_file(c_void_p(self._handle))
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


class _Stager:
    """A device buffer that tensors whose stored type differs from their device type pass through."""

    def __init__(self, device):
        self.device = device
        self.buf: Optional[torch.Tensor] = None

    def get(self, nbytes: int) -> torch.Tensor:
        if self.buf is None or self.buf.numel() < nbytes:
            self.buf = None
            self.buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        return self.buf


def _check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what}: error {code}")


class FileSource:
    """The tensors of a model folder's safetensors files, copied from pinned mappings."""

    def __init__(self, model_dir: str, register: bool = True):
        from .safetensors_io import SafetensorsError, open_model_files
        self.model_dir = model_dir
        self.files = open_model_files(model_dir)
        self.register = register
        self.where: Dict[str, object] = {}
        self.available: Dict[str, Tuple[Tuple[int, ...], torch.dtype]] = {}
        for f in self.files:
            for name, ent in f.entries.items():
                if name in self.available:
                    self.close()
                    raise SafetensorsError(f"tensor '{name}' appears in more than one shard")
                self.available[name] = (ent.shape, ent.dtype)
                self.where[name] = f
        self.pinned_files = 0
        self.bytes_copied = 0

    def close(self) -> None:
        for f in self.files:
            f.close()

    def fill(self, arena: WeightArena, names: Iterable[str]) -> None:
        """Copy every tensor of ``names`` into its place.  Returns when all copies have landed."""
        lib = _lib()
        dev = arena.device
        maps: Dict[str, MappedFile] = {}
        stream = torch.cuda.Stream(device=dev)
        stager = _Stager(dev)
        sp = c_void_p(stream.cuda_stream)
        try:
            with torch.cuda.device(dev):
                for name in names:
                    f = self.where[name]
                    ent = f.entries[name]
                    if f.path not in maps:
                        maps[f.path] = MappedFile(f.path, self.register)
                    m = maps[f.path]
                    dst, pl = arena.destination(name)
                    rows, cols = _rows_cols(ent.shape)
                    if rows * cols == 0:
                        continue
                    src_addr = m.address + ent.begin
                    es = ent.end - ent.begin
                    self.bytes_copied += es
                    if not ent.dtype.is_floating_point:
                        if pl.slot != name:
                            raise ValueError(f"integer tensor '{name}' cannot be part of a fused tensor")
                        # integer tables are small: widened or narrowed to int32 on the host
                        t = f.tensor(name).to(torch.int32).contiguous()
                        stream.synchronize()
                        dst.view(-1)[pl.row0 * cols: pl.row0 * cols + t.numel()].copy_(t.view(-1))
                        continue
                    if ent.dtype == dst.dtype:
                        _check(lib.ff_weights_copy_rows(c_void_p(dst.data_ptr()), c_void_p(src_addr), c_longlong(rows),
                                                        c_longlong(cols * dst.element_size()), c_longlong(pl.row0),
                                                        c_longlong(pl.group), c_longlong(pl.group_stride), sp),
                               f"copy of '{name}'")
                        continue
                    # another stored type: raw bytes to the staging buffer, conversion into place, in
                    # pieces of whole groups of rows
                    src_es = es // (rows * cols)
                    per = max(pl.group, (STAGING_BYTES // (cols * src_es)) // pl.group * pl.group)
                    stage = stager.get(min(rows, per) * cols * src_es)
                    for r0 in range(0, rows, per):
                        n = min(per, rows - r0)
                        _check(lib.ff_weights_copy_rows(c_void_p(stage.data_ptr()),
                                                        c_void_p(src_addr + r0 * cols * src_es), c_longlong(1),
                                                        c_longlong(n * cols * src_es), c_longlong(0), c_longlong(1),
                                                        c_longlong(1), sp), f"copy of '{name}'")
                        _check(lib.ff_weights_convert_rows(
                            c_void_p(stage.data_ptr()), c_int(_WT[ent.dtype]), c_void_p(dst.data_ptr()),
                            c_int(_WT[dst.dtype]), c_longlong(n), c_longlong(cols),
                            c_longlong(pl.row0 + (r0 // pl.group) * pl.group_stride), c_longlong(pl.group),
                            c_longlong(pl.group_stride), sp), f"conversion of '{name}'")
                stream.synchronize()
        finally:
            stream.synchronize()
            self.pinned_files = sum(1 for m in maps.values() if m.pinned)
            for m in maps.values():
                m.close()
            if stager.buf is not None:
                stager.buf = None
                torch.cuda.empty_cache()


class RandomSource:
    """Seeded random tensors drawn on the device into their places (see ``random_init``)."""

    def __init__(self, specs, seed: int, stored: torch.dtype = torch.float32):
        """``stored``: the type a checkpoint of these weights would hold them in; a value is rounded to
        it once, also where the device keeps the tensor in a wider type."""
        self.specs = {w.name: w for w in specs}
        self.seed = seed
        self.stored = stored

    def fill(self, arena: WeightArena, names: Iterable[str]) -> None:
        from . import random_init as R
        lib = _lib()
        dev = arena.device
        with torch.cuda.device(dev):
            table = R.normal_table().to(dev)
            sp = c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            for name in names:
                w = self.specs[name]
                dst, pl = arena.destination(name)
                rows, cols = _rows_cols(w.shape)
                if rows * cols == 0:
                    continue
                key = R.tensor_key(self.seed, name)
                if w.kind == "int":
                    if pl.slot != name:
                        raise ValueError(f"integer tensor '{name}' cannot be part of a fused tensor")
                    _check(lib.ff_weights_random_ints(c_void_p(dst.data_ptr()), c_longlong(rows * cols), c_ulonglong(key),
                                                      c_ulonglong(R.int_high(w)), sp), f"random '{name}'")
                    continue
                scale, shift = R.law(w)
                _check(lib.ff_weights_random_rows(c_void_p(dst.data_ptr()), c_int(_WT[dst.dtype]), c_longlong(rows),
                                                  c_longlong(cols), c_longlong(pl.row0), c_longlong(pl.group),
                                                  c_longlong(pl.group_stride), c_ulonglong(key),
                                                  c_void_p(table.data_ptr()), c_float(scale), c_float(shift),
                                                  c_int(1 if self.stored == torch.bfloat16 else 0), sp),
                       f"random '{name}'")
            torch.cuda.synchronize(dev)
