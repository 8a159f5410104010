"""The peer-store exchange of the column-sharded decode step (include/llmp_b200.h, "peer
exchange"): buffers every rank can store into, their flag words, and the calls over them.

One process a GPU.  `PeerExchange` allocates this rank's buffers through the library (an
exportable allocation must be a whole one, so these do not come from torch's allocator),
exports them as CUDA IPC handles (the caller trades those, e.g. with torch.distributed's
all_gather_object) and keeps the device tables the kernels read.  Buffers are seen as torch tensors through the CUDA array interface."""
from __future__ import annotations

import ctypes as C

import torch

from . import _native as N

DEFAULT_POLLS = 1 << 22      # x about 0.1 us: a wait gives up after roughly half a second


class _Device:
    """A library allocation as an object torch.as_tensor can wrap."""

    def __init__(self, ptr: int, shape: tuple[int, ...], typestr: str):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False),
                                         "version": 2}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class PeerExchange:
    """`vectors`: name -> F32 length of a gathered vector.  `sites`: exchanges a step.
    Construct on every rank, trade `handles()` (or, for ranks emulated inside one process,
    `pointers()`), then `connect()`."""

    def __init__(self, world: int, rank: int, vectors: dict[str, int], sites: int,
                 words: dict[str, int] | None = None):
        """`words`: name -> length of a vector of tagged 8-byte words (the in-band form)."""
        self.world, self.rank, self.sites = world, rank, sites
        self._owned, self._opened = [], []
        words = words or {}
        self._names = list(vectors) + list(words)
        self._local = {name: self._alloc(vectors[name] * 4) for name in vectors}
        self._local.update({name: self._alloc(words[name] * 8) for name in words})
        self.words = {name: torch.as_tensor(_Device(self._local[name], (words[name],), "<i8"),
                                            device="cuda") for name in words}
        self._local_flags = self._alloc(sites * world * 4)
        self._step = self._alloc(256)
        self._status = self._alloc(256)
        self._tables, self._flag_table = {}, None
        self.vectors = {name: torch.as_tensor(_Device(self._local[name], (vectors[name],), "<f4"),
                                              device="cuda") for name in vectors}
        self.status = torch.as_tensor(_Device(self._status, (1,), "<i4"), device="cuda")
        self.step = torch.as_tensor(_Device(self._step, (1,), "<i4"), device="cuda")

    def _alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        N.check(N.lib().llmp_b200_peer_alloc(nbytes, C.byref(p)), "llmp_b200_peer_alloc")
        self._owned.append(p.value)
        return p.value

    def pointers(self) -> dict[str, int]:
        """This rank's buffers as addresses: for ranks that share this process."""
        return {"flags": self._local_flags, **self._local}

    def handles(self) -> dict[str, bytes]:
        """This rank's buffers as CUDA IPC handles: for ranks in other processes."""
        def export(ptr: int) -> bytes:
            h = (C.c_ubyte * 64)()
            N.check(N.lib().llmp_b200_peer_export(ptr, h), "llmp_b200_peer_export")
            return bytes(h)
        return {key: export(ptr) for key, ptr in self.pointers().items()}

    def connect(self, everyone: list[dict]) -> None:
        """everyone[r]: rank r's handles() or pointers()."""
        if len(everyone) != self.world:
            raise N.Rejected("peer exchange: one entry a rank")

        def open_(entry) -> int:
            if isinstance(entry, int):
                return entry
            h = (C.c_ubyte * 64).from_buffer_copy(entry)
            p = C.c_void_p()
            N.check(N.lib().llmp_b200_peer_import(h, C.byref(p)), "llmp_b200_peer_import")
            self._opened.append(p.value)
            return p.value

        def table(key: str, own: int) -> torch.Tensor:
            ptrs = [own if r == self.rank else open_(everyone[r][key]) for r in range(self.world)]
            return torch.tensor(ptrs, dtype=torch.int64, device="cuda")

        self._tables = {name: table(name, self._local[name]) for name in self._names}
        self._flag_table = table("flags", self._local_flags)

    def _site(self, name: str, site: int) -> N.PeerSite:
        if not 0 <= site < self.sites:
            raise N.Rejected(f"peer exchange: site {site} of {self.sites}")
        s = N.PeerSite()
        s.world, s.rank, s.site = self.world, self.rank, site
        s.buffers, s.flags = self._tables[name].data_ptr(), self._flag_table.data_ptr()
        s.step = self._step
        return s

    def begin_step(self) -> None:
        N.check(N.lib().llmp_b200_peer_begin_step(self._step, _stream()), "llmp_b200_peer_begin_step")

    def publish(self, name: str, site: int, piece: torch.Tensor, offset_floats: int) -> None:
        """This rank's slice (F32, contiguous, the stream's last output) into every rank's copy."""
        if piece.dtype != torch.float32 or not piece.is_contiguous():
            raise N.Rejected("peer publish: a contiguous F32 slice")
        s = self._site(name, site)
        N.check(N.lib().llmp_b200_peer_publish(C.byref(s), piece.data_ptr(), offset_floats * 4,
                                               piece.numel() * 4, _stream()), "llmp_b200_peer_publish")

    def wait(self, name: str, site: int, polls: int = DEFAULT_POLLS) -> None:
        s = self._site(name, site)
        N.check(N.lib().llmp_b200_peer_wait(C.byref(s), self._local_flags, polls, self._status,
                                            _stream()), "llmp_b200_peer_wait")

    def quantize_q8(self, name: str, site: int, out: torch.Tensor, polls: int = DEFAULT_POLLS,
                    x: torch.Tensor | None = None) -> torch.Tensor:
        """Q8_1 blocks of the gathered vector `name` (or of `x`, F32 [k], when the exchange is
        waited for as back-pressure only), once every rank's slice of `site` arrived."""
        x = self.vectors[name] if x is None else x.reshape(-1)
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise N.Rejected("peer quantize: a contiguous F32 vector")
        s = self._site(name, site)
        N.check(N.lib().llmp_b200_q8_1_quantize_gathered(
            x.data_ptr(), x.numel(), 1, x.numel(), out.data_ptr(), C.byref(s), self._local_flags,
            polls, self._status, _stream()), "llmp_b200_q8_1_quantize_gathered")
        return out

    def exchange_quantize_q8(self, name: str, site: int, piece: torch.Tensor, offset_floats: int,
                             out: torch.Tensor, polls: int = DEFAULT_POLLS,
                             x: torch.Tensor | None = None) -> torch.Tensor:
        """publish() + quantize_q8() as one launch."""
        if piece.dtype != torch.float32 or not piece.is_contiguous():
            raise N.Rejected("peer exchange: a contiguous F32 slice")
        x = self.vectors[name] if x is None else x.reshape(-1)
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise N.Rejected("peer exchange: a contiguous F32 vector")
        s = self._site(name, site)
        N.check(N.lib().llmp_b200_q8_1_quantize_exchange(
            x.data_ptr(), x.numel(), out.data_ptr(), C.byref(s), self._local_flags,
            piece.data_ptr(), offset_floats * 4, piece.numel() * 4, polls, self._status, _stream()),
            "llmp_b200_q8_1_quantize_exchange")
        return out

    # ---- the in-band form: values as tagged words, stored by the product kernel itself
    def fan(self, name: str, base: int, tag: int) -> N.PeerFan:
        """For ops.vecq(..., fan=): token 0's results also go to words[base + row] of every rank."""
        f = N.PeerFan()
        f.world, f.words, f.step = self.world, self._tables[name].data_ptr(), self._step
        f.base, f.tag = base, tag
        return f

    def quantize_words(self, out: torch.Tensor, *, name: str | None = None, first: int = 0,
                       count: int = 0, tag: int = 0, x: torch.Tensor | None = None,
                       hold: tuple[str, int, int, int] | None = None,
                       polls: int = DEFAULT_POLLS) -> torch.Tensor:
        """Q8_1 blocks of words[name][first:first + count] once they carry `tag`, or of `x` (F32);
        `hold` = (name, first, count, tag): words waited for first, values unused."""
        L = N.lib()
        if (x is None) == (name is None):
            raise N.Rejected("peer quantize_words: either a word vector or x")
        if x is not None:
            x = x.reshape(-1)
            if x.dtype != torch.float32 or not x.is_contiguous():
                raise N.Rejected("peer quantize_words: a contiguous F32 vector")
            k, words_ptr, x_ptr = x.numel(), None, x.data_ptr()
        else:
            k, words_ptr, x_ptr = count, self._local[name] + (first * 8), None
        hold_ptr, hold_count, hold_tag = None, 0, 0
        if hold is not None:
            hold_ptr, hold_count, hold_tag = self._local[hold[0]] + (hold[1] * 8), hold[2], hold[3]
        N.check(L.llmp_b200_q8_1_quantize_words(x_ptr, words_ptr, tag, k, hold_ptr, hold_count,
                                                hold_tag, self._step, out.data_ptr(), polls,
                                                self._status, _stream()),
                "llmp_b200_q8_1_quantize_words")
        return out

    def word_values(self, name: str, first: int, count: int) -> torch.Tensor:
        """The F32 values of a run of words (their low halves)."""
        return self.words[name][first:first + count].view(torch.int32)[::2].contiguous().view(torch.float32)

    def timed_out(self) -> bool:
        """Whether a wait of this rank ran out since the last call (reads the device word)."""
        hit = int(self.status.item()) != 0
        self.status.zero_()
        return hit

    def close(self) -> None:
        torch.cuda.synchronize()
        L = N.lib()
        for p in self._opened:
            L.llmp_b200_peer_close(p)
        for p in self._owned:
            L.llmp_b200_peer_free(p)
        self._opened, self._owned = [], []
