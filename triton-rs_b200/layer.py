"""Host-side handle for the decode-layer chain (`b200k_layer_*` in the C ABI), and the
tensor-parallel sharding of its int4 weights.

The class only owns device memory (through torch) and forwards to the library; the
sharding helpers are pure index arithmetic on the packed tensors.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from ._lib import lib


class _Config(ctypes.Structure):
    _fields_ = [("hidden", ctypes.c_int), ("num_q_heads", ctypes.c_int), ("num_kv_heads", ctypes.c_int),
                ("head_dim", ctypes.c_int), ("intermediate", ctypes.c_int), ("group_size", ctypes.c_int),
                ("weight_format", ctypes.c_int), ("max_batch", ctypes.c_int), ("max_len", ctypes.c_int),
                ("rms_eps", ctypes.c_float), ("use_graph", ctypes.c_int), ("reserved", ctypes.c_int * 5)]


@dataclass
class LayerShape:
    """Extents of one decode layer (global, before any tensor-parallel split)."""
    hidden: int = 4096
    num_q_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 14336
    group_size: int = 128
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0

    def local(self, world: int) -> "LayerShape":
        assert self.num_q_heads % world == 0 and self.num_kv_heads % world == 0 and self.intermediate % world == 0
        assert (self.intermediate // world) % self.group_size == 0
        return LayerShape(self.hidden, self.num_q_heads // world, self.num_kv_heads // world, self.head_dim,
                          self.intermediate // world, self.group_size, self.rms_eps, self.rope_theta)


# ---- tensor-parallel sharding of packed int4 weights -------------------------------
def _cols(t, lo, hi, per_word):
    """Column slice [lo, hi) of a tensor whose last axis packs `per_word` columns per element."""
    assert lo % per_word == 0 and hi % per_word == 0
    return t[..., lo // per_word: hi // per_word]


def shard_columns(w, blocks, rank, world, fmt="gptq"):
    """Column-parallel shard of (qweight, scales, qzeros).  `blocks` lists the widths of the
    fused sub-blocks along N (e.g. [Hq*D, Hkv*D, Hkv*D] for QKV, [I, I] for gate|up); each
    sub-block is split separately so that a rank's q/k/v heads and gate/up pairs stay together."""
    qw, sc, qz = w
    qw_per = 1 if fmt == "gptq" else 8
    parts_q, parts_s, parts_z = [], [], []
    off = 0
    for width in blocks:
        assert width % world == 0
        lo = off + rank * (width // world)
        hi = lo + width // world
        parts_q.append(_cols(qw, lo, hi, qw_per))
        parts_s.append(sc[..., lo:hi])
        if qz is not None:
            parts_z.append(_cols(qz, lo, hi, 8))
        off += width
    cat = lambda ps: torch.cat(ps, dim=-1).contiguous()
    return cat(parts_q), cat(parts_s), (cat(parts_z) if qz is not None else None)


def shard_rows(w, rank, world, group_size, fmt="gptq"):
    """Row-parallel shard (split K; boundaries on quantisation groups)."""
    qw, sc, qz = w
    k = qw.shape[0] * (8 if fmt == "gptq" else 1)
    assert k % world == 0 and (k // world) % group_size == 0
    lo, hi = rank * (k // world), (rank + 1) * (k // world)
    rows_per = 8 if fmt == "gptq" else 1
    return (qw[lo // rows_per: hi // rows_per].contiguous(), sc[lo // group_size: hi // group_size].contiguous(),
            None if qz is None else qz[lo // group_size: hi // group_size].contiguous())


def shard_layer_weights(weights, shape: LayerShape, rank, world, fmt="gptq"):
    """weights: dict qkv/o/gate_up/down -> (qweight, scales, qzeros) for the whole layer."""
    d = shape.head_dim
    return {
        "qkv": shard_columns(weights["qkv"], [shape.num_q_heads * d, shape.num_kv_heads * d, shape.num_kv_heads * d],
                             rank, world, fmt),
        "o": shard_rows(weights["o"], rank, world, shape.group_size, fmt),
        "gate_up": shard_columns(weights["gate_up"], [shape.intermediate, shape.intermediate], rank, world, fmt),
        "down": shard_rows(weights["down"], rank, world, shape.group_size, fmt),
    }


class Comm:
    """Exchange buffer of one tensor-parallel rank for the library's peer-to-peer all-reduce.

    `exchange(handle: bytes) -> list[bytes]` must return the 64-byte handles of all ranks in rank order
    (an all-gather between the processes, one per GPU, of one node)."""

    def __init__(self, rank: int, world: int, slot_bytes: int, exchange):
        self._L = lib()
        self.rank, self.world, self.slot_bytes = rank, world, slot_bytes
        handle = ctypes.c_void_p()
        self._L.call("b200k_comm_create", rank, world, slot_bytes, ctypes.addressof(handle))
        self.handle = handle.value
        mine = ctypes.create_string_buffer(64)
        self._L.call("b200k_comm_ipc_handle", self.handle, ctypes.addressof(mine))
        handles = [bytes(mine.raw)] if world == 1 else list(exchange(bytes(mine.raw)))
        if len(handles) != world or any(len(h) != 64 for h in handles):
            raise ValueError("exchange() must return one 64-byte handle per rank")
        blob = ctypes.create_string_buffer(b"".join(handles), 64 * world)
        self._L.call("b200k_comm_open_peers", self.handle, ctypes.addressof(blob))

    @classmethod
    def from_process_group(cls, slot_bytes: int, group=None):
        """One rank per GPU over an initialised torch.distributed process group (handles travel as
        Python objects through the group's all-gather)."""
        import torch.distributed as dist

        def exchange(h):
            out = [None] * dist.get_world_size(group)
            dist.all_gather_object(out, h, group=group)
            return out
        return cls(dist.get_rank(group), dist.get_world_size(group), slot_bytes, exchange)

    def slot(self, slot: int) -> int:
        """Device address of slot 0 or 1 of this rank's buffer."""
        p = ctypes.c_void_p()
        self._L.call("b200k_comm_slot", self.handle, slot, ctypes.addressof(p))
        return p.value

    def all_reduce(self, slot: int, output, count: int, input=None, stream=None):
        st = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        self._L.call("b200k_comm_allreduce_f16", self.handle, slot, input, output, count, st)
        return output

    def status(self) -> int:
        v = ctypes.c_int(-1)
        self._L.call("b200k_comm_status", self.handle, ctypes.addressof(v), torch.cuda.current_stream().cuda_stream)
        return v.value

    def close(self):
        if self.handle:
            self._L.raw("b200k_comm_destroy")(self.handle)
            self.handle = None


class DecodeLayer:
    """One decode layer on one GPU (one tensor-parallel rank)."""
    ORDER = ("qkv", "o", "gate_up", "down")

    def __init__(self, shape: LayerShape, weights, ln1, ln2, cos, sin, max_batch, max_len, fmt="gptq",
                 use_graph=True, k_cache=None, v_cache=None):
        self.shape, self.max_batch, self.max_len = shape, max_batch, max_len
        self._L = lib()
        cfg = _Config(shape.hidden, shape.num_q_heads, shape.num_kv_heads, shape.head_dim, shape.intermediate,
                      shape.group_size, 0 if fmt == "gptq" else 1, max_batch, max_len, shape.rms_eps,
                      1 if use_graph else 0)
        handle = ctypes.c_void_p()
        self._L.call("b200k_layer_create", ctypes.addressof(cfg), ctypes.addressof(handle))
        self.handle = handle.value
        self._keep = [weights, ln1, ln2, cos, sin]       # the library does not copy these
        for i, name in enumerate(self.ORDER):
            qw, sc, qz = weights[name]
            self._L.call("b200k_layer_set_weight", self.handle, i, qw, sc, qz)
        self._L.call("b200k_layer_set_norms_rope", self.handle, ln1, ln2, cos, sin)
        dev = ln1.device
        if k_cache is None:
            k_cache = torch.zeros((max_batch, shape.num_kv_heads, max_len, shape.head_dim), dtype=torch.float16, device=dev)
            v_cache = torch.zeros_like(k_cache)
        self.k_cache, self.v_cache = k_cache, v_cache
        self._L.call("b200k_layer_set_kv_cache", self.handle, k_cache, v_cache)

    def set_kv_cache(self, k_cache, v_cache):
        self.k_cache, self.v_cache = k_cache, v_cache
        self._L.call("b200k_layer_set_kv_cache", self.handle, k_cache, v_cache)

    def set_comm(self, comm: "Comm | None"):
        """Attach the exchange buffer: forward() then runs the two all-reduces of a tensor-parallel layer itself."""
        self.comm = comm
        self._L.call("b200k_layer_set_comm", self.handle, comm.handle if comm is not None else None)

    def _stream(self, stream):
        return stream if stream is not None else torch.cuda.current_stream().cuda_stream

    def forward(self, hidden, positions, out=None, stream=None):
        out = torch.empty_like(hidden) if out is None else out
        self._L.call("b200k_layer_forward", self.handle, hidden, positions, out, hidden.shape[0], self._stream(stream))
        return out

    def forward_host(self, host_hidden, host_positions, host_out, stream=None):
        """host_* are pinned CPU tensors; returns after enqueueing (synchronise the stream to read host_out)."""
        self._L.call("b200k_layer_forward_host", self.handle, host_hidden.data_ptr(), host_positions.data_ptr(),
                     host_out.data_ptr(), host_hidden.shape[0], self._stream(stream))
        return host_out

    def forward_stage(self, stage, hidden=None, positions=None, reduced=None, partial=None, out=None, batch=None,
                      stream=None):
        self._L.call("b200k_layer_forward_stage", self.handle, stage, hidden, positions, reduced, partial, out, batch,
                     self._stream(stream))

    @property
    def launches_per_forward(self):
        return self._L.call("b200k_layer_launches_per_forward", self.handle)

    def close(self):
        if self.handle:
            self._L.raw("b200k_layer_destroy")(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
