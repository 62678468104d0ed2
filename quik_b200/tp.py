"""Tensor-parallel column split of a MixedQLinear over the ranks of a torch.distributed group.

The layer shards naturally by output channel: rank r holds rows [r*N/g, (r+1)*N/g) of int_weight,
fp_weight, weights_scales and reduced_w; the activations are replicated and every rank runs the
(cheap) quantizer itself, so no broadcast sits on the critical path.  The only exchange is the
assembly of the [M, N] output from the g slabs [M, N/g].  The reference has no multi-GPU path for
the layer (experiments/llama.py:295-326 only places whole layers on different GPUs).

Two ways to assemble:

``mode="pull"`` (default on NVLink machines): the row-major [M, N] result of every rank lives in
symmetric memory and the rank's fused kernel writes its own column range into it in place (output
row pitch N).  After a stream-ordered barrier each rank pulls the g-1 remote column ranges from the
peers' buffers into the same ranges of its own with strided copies on the copy engines
(``quik_copy_2d``), one stream per peer so that several copy engines work at once (the streams are shared
by all layers of a device: the assemblies of successive layers run one after the other).  No SM time, no
staging buffer, no permute pass, no local copy, and the transfer of layer i overlaps the kernels of
the layers after it.  The result alternates between two symmetric buffers, which makes one barrier
per forward enough: a rank overwrites its column range of a buffer two forwards later, after it has
passed the barrier of the forward in between -- and a peer reaches that barrier only when its pulls
of the earlier forward are complete.  A layer whose assembled output is large runs as ``chunks`` blocks
of token rows (the layer is row-independent: per-token quantization, so the values do not change): the
pulls of a block start while the kernels of the next block run, so most of the transfer hides behind the
layer's own computation instead of starting after it.

``mode="nccl"``: ``all_gather_into_tensor`` of the slabs followed by a permute to row-major (also
the path used on CPU/gloo in the tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


_STREAMS = {}      # (device index, world size) -> {"comm": stream, "peers": [stream per peer]}


def shard_range(n_total: int, world: int, rank: int, multiple: int = 8) -> slice:
    """Contiguous, equal-sized shard of the output channels (n_total must divide evenly)."""
    if n_total % (world * multiple) != 0:
        raise ValueError(f"out_features={n_total} does not split into {world} shards that are multiples of {multiple}")
    per = n_total // world
    return slice(rank * per, (rank + 1) * per)


class ColumnParallelMixedQLinear(torch.nn.Module):
    """Wraps the local shard (a MixedQLinear over N/g output channels) and assembles the full output.

    ``forward`` returns the [1, M, N] result; in pull mode the tensor is complete once ``wait()`` has
    been called (or the side stream has been joined by other means) -- the copies run on ``comm_stream``.
    """

    # chunks=None: cut the layer into row blocks when a rank pulls more than CHUNK_BYTES per block.  Not the default:
    # on 4 GPUs the 70B step measured 1.30 ms with whole layers, 1.37 ms with two and 1.44 ms with four blocks (smaller
    # GEMMs lose more to their last wave than the earlier start of the pulls gains)
    CHUNK_BYTES = 48 << 20
    MAX_CHUNKS = 4
    # copy="auto" pulls column ranges narrower than SM_COPY_BELOW bytes with a copy kernel (quik_copy_2d_sm: small CTAs
    # that fit beside the layer kernels) instead of the copy engines.  Not the default: on 8 GPUs (70B shapes, 2-2.5 KB
    # per row and rank in three of the four layers) the assembly alone went from 1.74 to 1.64 ms, but the step from 1.91
    # to 1.99 ms (the copy CTAs take issue slots from the layer kernels); on 4 GPUs the two measured alike.
    SM_COPY_BELOW = 8192
    SM_COPY_CTAS = 64

    def __init__(self, local: torch.nn.Module, group=None, gather_output: bool = True, mode: str = "nccl",
                 comm_stream=None, chunks=1, copy="ce"):
        super().__init__()
        self.local = local
        self.group = group if group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.gather_output = gather_output
        self.world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        self.mode = mode
        self.comm_stream = comm_stream
        self.copy = copy           # "ce": copy engines; "sm": copy kernel; "auto": the kernel for rows below SM_COPY_BELOW
        self.chunks = chunks       # row blocks per forward in pull mode (1 = whole layer); None = by the size of the output
        self._bufs = []            # two symmetric [M, N] results, used in turn
        self._hdls = []
        self._turn = 0
        self._peer_streams = []
        self._passed = None        # event: the barrier of the last forward has been passed on the comm stream
        self._done = None          # event: assembly of the last forward finished
        self._last = None          # result tensor of the last forward

    # ---- pull mode ---------------------------------------------------------------------------
    def _setup_pull(self, m, n_local, dtype, device):
        import torch.distributed._symmetric_memory as symm_mem
        n = n_local * self.world
        # the whole [M, N] result lives in symmetric memory; the local fused kernel writes its column
        # range in place (row pitch N), the peers read that range from here
        self._bufs, self._hdls = [], []
        for _ in range(2):
            full = symm_mem.empty((m, n), dtype=dtype, device=device)
            self._hdls.append(symm_mem.rendezvous(full, self.group))
            self._bufs.append(full)
        self._turn = 0
        # one assembly stream and one stream per peer for all layers of a device: the assemblies of successive layers
        # run one after the other at the link's rate (several at once, each with its own streams, measured 410 GB/s
        # per rank against 490-670 GB/s one at a time on 4 GPUs)
        shared = _STREAMS.setdefault((device.index, self.world), {})
        if not shared:
            shared["comm"] = torch.cuda.Stream(device=device)
            shared["peers"] = [torch.cuda.Stream(device=device) for _ in range(self.world - 1)]
        if self.comm_stream is None:
            self.comm_stream = shared["comm"]
        self._peer_streams = shared["peers"]

    def _forward_pull(self, x):
        m = x.shape[-2]
        n_local = self.local.out_features
        if not self._bufs or self._bufs[0].shape[0] != m:
            self._setup_pull(m, n_local, x.dtype, x.device)
        b = self._turn & 1
        self._turn += 1
        full, hdl = self._bufs[b], self._hdls[b]
        cur = torch.cuda.current_stream(x.device)
        if self._passed is not None:
            # this buffer was last used two forwards ago; every peer finished pulling from it before it arrived at
            # the barriers of the forward in between, which this rank has passed once this event has fired
            cur.wait_event(self._passed)
        width = n_local * full.element_size()
        x2 = x.reshape(-1, x.shape[-1])
        for r0, r1 in self._row_blocks(m, width):
            slab = full[r0:r1, self.rank * n_local:(self.rank + 1) * n_local]
            self.local.out_buffer = slab
            out = self.local(x2[r0:r1].unsqueeze(0))     # writes its column range of these rows of `full`
            assert out.data_ptr() == slab.data_ptr(), "local layer did not write into the symmetric buffer"
            ready = torch.cuda.Event()
            ready.record(cur)
            self._assemble(full, hdl, r0, r1, n_local, ready)
        self._last = full
        return full.unsqueeze(0)

    def _assemble(self, full, hdl, r0, r1, n_local, ready):
        """On the comm stream: wait for `ready` (this rank's column range of rows [r0, r1) is written), meet the peers
        at a barrier, pull their column ranges of those rows."""
        from ._lib import check, load
        lib = load()
        width = n_local * full.element_size()
        pitch = full.shape[1] * full.element_size()
        comm = self.comm_stream
        with torch.cuda.stream(comm):
            comm.wait_event(ready)
            hdl.barrier(channel=0)               # every rank's column range of these rows is complete
            passed = torch.cuda.Event()
            passed.record(comm)
            joins = []
            for step in range(1, self.world):
                peer = (self.rank + step) % self.world      # walk the ring so the links load evenly
                src = hdl.get_buffer(peer, tuple(full.shape), full.dtype)
                off = r0 * pitch + peer * width
                ps = self._peer_streams[step - 1]
                ps.wait_event(passed)
                if self.copy == "sm" or (self.copy == "auto" and width < self.SM_COPY_BELOW and width % 16 == 0):
                    check(lib.quik_copy_2d_sm(full.data_ptr() + off, pitch, src.data_ptr() + off, pitch, width, r1 - r0,
                                              self.SM_COPY_CTAS, ps.cuda_stream), "quik_copy_2d_sm")
                else:
                    check(lib.quik_copy_2d(full.data_ptr() + off, pitch, src.data_ptr() + off, pitch, width, r1 - r0,
                                           ps.cuda_stream), "quik_copy_2d")
                ev = torch.cuda.Event()
                ev.record(ps)
                joins.append(ev)
            for ev in joins:
                comm.wait_event(ev)              # the comm stream reaches its next barrier only after these pulls
            self._passed = passed
            self._done = torch.cuda.Event()
            self._done.record(comm)

    def assemble_again(self):
        """Repeat the assembly of the last forward's buffer without running the layer (to time the transfer alone).
        Returns the bytes this rank pulls."""
        if self._last is None:
            return 0
        b = (self._turn - 1) & 1
        full, hdl = self._bufs[b], self._hdls[b]
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(full.device))
        self._assemble(full, hdl, 0, full.shape[0], self.local.out_features, ready)
        return full.shape[0] * self.local.out_features * full.element_size() * (self.world - 1)

    def _row_blocks(self, m, width_bytes):
        """Row ranges of one forward: one block, or up to MAX_CHUNKS equal blocks of a multiple of 256 rows when the
        bytes this rank pulls exceed CHUNK_BYTES per block."""
        c = self.chunks
        if c is None:
            pulled = m * width_bytes * (self.world - 1)
            c = max(1, min(self.MAX_CHUNKS, pulled // self.CHUNK_BYTES))
        c = max(1, min(int(c), m // 256 if m >= 256 else 1))
        rows = -(-m // c)
        rows = -(-rows // 256) * 256 if c > 1 else m
        return [(r0, min(m, r0 + rows)) for r0 in range(0, m, rows)]

    def reset(self):
        """Forget the events of earlier forwards (call before capturing a CUDA graph, with the device idle)."""
        self._done = None
        self._passed = None

    def wait(self):
        """Make the current stream wait for the assembly of the last forward."""
        if self._done is not None:
            torch.cuda.current_stream().wait_event(self._done)

    # ---- forward -----------------------------------------------------------------------------
    def forward(self, x):
        if self.world == 1 or not self.gather_output:
            return self.local(x)
        if self.mode == "pull":
            return self._forward_pull(x)
        out = self.local(x)                                  # [1, M, N/g]
        m, n_local = out.shape[1], out.shape[2]
        slabs = torch.empty((self.world * m, n_local), dtype=out.dtype, device=out.device)
        dist.all_gather_into_tensor(slabs, out[0].contiguous(), group=self.group)
        # [g, M, N/g] -> row-major [M, N]
        return slabs.view(self.world, m, n_local).permute(1, 0, 2).reshape(1, m, self.world * n_local)
