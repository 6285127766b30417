"""Tensor-parallel use of the SpMM: how one layer's weights are split over the GPUs of a box.

The reference itself is single-GPU; its weight-conversion tool shards every layer offline and
FasterTransformer adds the collective (end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:134-135:
QKV and FFN1 are split by output rows M, out-proj and FFN2 by K).  The same two splits here:

* column-parallel (by rows of A): tiles are emitted row-of-tiles major (csrc/SpMM_API.cu:313-314),
  so the rows of rank r are a contiguous slice of the words and offsets of the whole matrix --
  `row_shard` cuts it out, bit-identical to encoding the shard alone.  B is replicated, every rank
  produces its own rows of C, no collective.
* row-parallel (by K): rank r owns columns [r*K/g, (r+1)*K/g) of A and the matching rows of B.  The
  columns are not contiguous in the encoded stream, so each shard is encoded from its dense slice
  (`column_slice`).  Every rank produces a full-size partial C; one sum all-reduce finishes it.

One process per GPU; `torch.distributed` (NCCL on GPUs, gloo in the CPU tests) carries the reduce.
"""
import numpy as np

TILE_M = 128
TILE_K = 64


def row_shard(words, offsets, M, K, rank, world):
    """Words and offsets of rows [rank*M/world, (rank+1)*M/world) cut from the encoding of the whole matrix.

    Returns (words, offsets, M_shard).  M/world must be a multiple of 128."""
    if M % (world * TILE_M) != 0:
        raise ValueError("M / world must be a multiple of %d" % TILE_M)
    tiles_k = K // TILE_K
    rows_of_tiles = M // TILE_M // world
    t0, t1 = rank * rows_of_tiles * tiles_k, (rank + 1) * rows_of_tiles * tiles_k
    offs = np.asarray(offsets[t0:t1 + 1], dtype=np.int64)
    shard_offsets = np.concatenate([offs - offs[0], [offs[-1] - offs[0]]]).astype(np.int32)  # duplicated tail entry
    shard_words = np.ascontiguousarray(words[int(offs[0]) * 4:int(offs[-1]) * 4])
    return shard_words, shard_offsets, rows_of_tiles * TILE_M


def column_slice(A, rank, world):
    """Dense columns [rank*K/world, (rank+1)*K/world) of A, contiguous, ready for the encoder."""
    K = A.shape[1]
    if K % (world * TILE_K) != 0:
        raise ValueError("K / world must be a multiple of %d" % TILE_K)
    k = K // world
    return np.ascontiguousarray(A[:, rank * k:(rank + 1) * k])


def activation_rows(B, rank, world):
    """Rows [rank*K/world, (rank+1)*K/world) of B[K][N]: the activations a row-parallel rank multiplies."""
    K = B.shape[0]
    k = K // world
    return np.ascontiguousarray(B[rank * k:(rank + 1) * k])


def all_reduce_partial(C_partial, group=None):
    """Sum of the ranks' partial results, in place.  C_partial: torch tensor (fp16 or fp32) on the
    device of the process group's backend."""
    import torch.distributed as dist
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(C_partial, op=dist.ReduceOp.SUM, group=group)
    return C_partial


class PeerAllReduce:
    """Sum of the ranks' fp16 partial results by the library's own kernel, which reads the peers'
    buffers over NVLink (csrc/allreduce_peer.cu) instead of calling a collective library.

    Holds two symmetric result buffers per rank (the SpMM of call n writes into `next_buffer()`, the
    kernel of call n reads all ranks' copies of it) and one symmetric flag array.  Every rank must
    construct it and call `reduce` the same number of times.  One process per GPU.

    `replayable=True` keeps the epoch in device memory so that `reduce` can be captured in a CUDA graph
    and replayed.  The buffer used by a call is then fixed at capture time (calls alternate between the
    two as usual), so a graph must either contain an even number of calls of this object or other
    exchanges among the same ranks between two of them (see include/spmm_b200.h)."""

    def __init__(self, count, device, group=None, replayable=False):
        import ctypes
        import os

        # plain peer mappings only: no NVLink multicast object is bound to these buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        from . import spmm_api
        self._api = spmm_api
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if count % 8:
            raise ValueError("count must be a multiple of 8 halves")
        self.count = count
        self.buffers = [symm_mem.empty(count, dtype=torch.float16, device=device) for _ in range(2)]
        self.flags = symm_mem.empty(64, dtype=torch.int32, device=device)
        self.flags.zero_()
        handles = [symm_mem.rendezvous(b, group) for b in self.buffers]
        flag_handle = symm_mem.rendezvous(self.flags, group)
        self._handles = handles + [flag_handle]  # keep the mappings alive
        ptr_array = ctypes.c_void_p * self.world
        self._buffer_ptrs = [ptr_array(*[int(p) for p in h.buffer_ptrs]) for h in handles]
        self._flag_ptrs = ptr_array(*[int(p) for p in flag_handle.buffer_ptrs])
        self.out = torch.empty(count, dtype=torch.float16, device=device)
        self.state = torch.zeros(2, dtype=torch.int32, device=device) if replayable else None
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group)  # nobody signals before every flag array is zero

    def next_buffer(self):
        """Where this rank's next partial result belongs (a view of the symmetric buffer)."""
        return self.buffers[(self.epoch + 1) & 1]

    def reduce(self, stream=None, limit_ms=2000):
        """Sums the partial results written into `next_buffer()` on every rank; returns the local sum."""
        import ctypes

        import torch
        if stream is None:
            stream = torch.cuda.current_stream()
        self.epoch += 1
        if self.state is not None:
            rc = self._api.LIB.spmm_b200_allreduce_partials_replayable(
                ctypes.c_void_p(stream.cuda_stream), self._buffer_ptrs[self.epoch & 1], self._flag_ptrs, self.rank, self.world,
                ctypes.c_void_p(self.out.data_ptr()), self.count, ctypes.c_void_p(self.state.data_ptr()), limit_ms)
        else:
            rc = self._api.LIB.spmm_b200_allreduce_partials(
                ctypes.c_void_p(stream.cuda_stream), self._buffer_ptrs[self.epoch & 1], self._flag_ptrs, self.rank, self.world,
                ctypes.c_void_p(self.out.data_ptr()), self.count, self.epoch, limit_ms)
        if rc != 0:
            raise RuntimeError("spmm_b200_allreduce_partials failed with cudaError %d" % rc)
        return self.out


class RowParallelSpMM:
    """One rank's part of a row-parallel layer on its GPU: SpMM over its K shard, then the sum over ranks,
    by NCCL (`reduce="nccl"`) or by the library's own peer-memory kernel (`reduce="peer"`)."""

    def __init__(self, words_dev, offsets_dev, M, N, K_shard, split_k=8, reduce="nccl", group=None, replayable=False):
        import torch
        from . import spmm_api
        self._api = spmm_api
        self.words, self.offsets = words_dev, offsets_dev
        self.M, self.N, self.K = M, N, K_shard
        self.split_k = split_k
        dev = words_dev.device
        self.C = torch.zeros((M, N), dtype=torch.float16, device=dev)
        self.workspace = torch.zeros(spmm_api.workspace_bytes(M, N, split_k) // 2, dtype=torch.int16, device=dev)
        self.peer = PeerAllReduce(M * N, dev, group, replayable=replayable) if reduce == "peer" else None

    def forward(self, B_shard_dev, group=None):
        C = self.peer.next_buffer() if self.peer is not None else self.C
        rc = self._api.SpMM_SplitK_API(None, None, self.words, None, None, self.offsets, B_shard_dev, C, self.M,
                                       self.N, self.K, self.workspace, self.split_k)
        if rc != 0:
            raise RuntimeError("SpMM_SplitK_API failed with cudaError %d" % rc)
        if self.peer is not None:
            return self.peer.reduce().view(self.M, self.N)
        return all_reduce_partial(self.C, group)


class FusedRowParallelSpMM:
    """One rank's part of a row-parallel layer with fp32 partial results summed over the ranks out of peer
    memory (spmm_b200_spmm_row_parallel): no collective library, one rounding, replayable from a CUDA graph.
    `fused=True`: the sum is folded into the SpMM kernel (one launch per call); `fused=False`: the SpMM only
    writes its fp32 partial rows and spmm_b200_allreduce_partials_f32 follows as a second launch (as fast,
    see include/spmm_b200.h).  Holds the symmetric partial buffers (two, used alternately), the
    symmetric flag array and the epoch state.  Every rank must construct it and call `forward` the same number
    of times.  With no process group (or a world of one) it runs stand-alone on one GPU."""

    def __init__(self, words_dev, offsets_dev, M, N, K_shard, split_k=8, group=None, fused=True, two_phase=False, announce=False):
        import ctypes

        import torch
        import torch.distributed as dist

        from . import spmm_api
        self._api = spmm_api
        self.words, self.offsets = words_dev, offsets_dev
        self.M, self.N, self.K, self.split_k = M, N, K_shard, split_k
        self.fused = fused
        # two_phase (with fused=False): spmm_b200_allreduce_partials_f32_two_phase -- every rank sums its share of
        # the rows and writes the result into all ranks' (symmetric) result buffers
        self.two_phase = bool(two_phase) and not fused
        # announce (with fused=False, two_phase=False): the SpMM's last block flags the partial rows to the peers
        # (partial_only = 2) and spmm_b200_allreduce_partials_f32_announced only waits and adds
        self.announce = bool(announce) and not fused and not two_phase
        dev = words_dev.device
        distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.rank = dist.get_rank(group) if distributed else 0
        self.world = dist.get_world_size(group) if distributed else 1
        flag_words = (M // TILE_M) * 4 * self.world
        ptr_array = ctypes.c_void_p * self.world
        if distributed:
            import os
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings only
            import torch.distributed._symmetric_memory as symm_mem
            group = group if group is not None else dist.group.WORLD
            self.partials = [symm_mem.empty(M * N, dtype=torch.float32, device=dev) for _ in range(2)]
            self.flags = symm_mem.empty(flag_words, dtype=torch.int32, device=dev)
            self.flags.zero_()
            handles = [symm_mem.rendezvous(b, group) for b in self.partials]
            flag_handle = symm_mem.rendezvous(self.flags, group)
            self._handles = handles + [flag_handle]  # keep the mappings alive
            if self.two_phase:
                if (M * N) % (8 * self.world) != 0:
                    raise ValueError("M * N must be a multiple of 8 * world for the two-phase sum")
                self.C = symm_mem.empty((M, N), dtype=torch.float16, device=dev)
                self.C.zero_()
                out_handle = symm_mem.rendezvous(self.C, group)
                self._handles.append(out_handle)
                self._out_ptrs = ptr_array(*[int(p) for p in out_handle.buffer_ptrs])
            self._partial_ptrs = (ctypes.c_void_p * (2 * self.world))(*[int(p) for h in handles for p in h.buffer_ptrs])
            self._flag_ptrs = ptr_array(*[int(p) for p in flag_handle.buffer_ptrs])
        else:
            self.partials = [torch.empty(M * N, dtype=torch.float32, device=dev) for _ in range(2)]
            self.flags = torch.zeros(flag_words, dtype=torch.int32, device=dev)
            self._partial_ptrs = (ctypes.c_void_p * 2)(self.partials[0].data_ptr(), self.partials[1].data_ptr())
            self._flag_ptrs = ptr_array(self.flags.data_ptr())
        self.state = torch.zeros(2, dtype=torch.int32, device=dev)
        if not (distributed and self.two_phase):
            self.C = torch.zeros((M, N), dtype=torch.float16, device=dev)
            self._out_ptrs = ptr_array(self.C.data_ptr()) if not distributed else None
        self.workspace = torch.zeros(spmm_api.workspace_bytes(M, N, split_k) // 2, dtype=torch.int16, device=dev)
        torch.cuda.synchronize(dev)
        if distributed:
            dist.barrier(group)  # nobody signals before every flag array is zero

    def forward(self, B_shard_dev, stream=None, limit_ms=2000, words=None):
        """`words`: another device copy of the same encoded weights to read this call (benchmarks rotate through
        copies to keep the weights out of L2); default: the tensor given at construction."""
        import ctypes

        import torch
        if stream is None:
            stream = torch.cuda.current_stream()
        words = self.words if words is None else words
        rc = self._api.LIB.spmm_b200_spmm_row_parallel(
            ctypes.c_void_p(stream.cuda_stream), ctypes.c_void_p(words.data_ptr()), ctypes.c_void_p(self.offsets.data_ptr()),
            ctypes.c_void_p(B_shard_dev.data_ptr()), ctypes.c_void_p(self.C.data_ptr()), self.M, self.N, self.K,
            ctypes.c_void_p(self.workspace.data_ptr()), self.split_k, self._partial_ptrs, self._flag_ptrs, self.rank, self.world,
            ctypes.c_void_p(self.state.data_ptr()), limit_ms, 0 if self.fused else (2 if self.announce else 1))
        if rc != 0:
            raise RuntimeError("spmm_b200_spmm_row_parallel failed with cudaError %d" % rc)
        if self.two_phase:
            rc = self._api.LIB.spmm_b200_allreduce_partials_f32_two_phase(
                ctypes.c_void_p(stream.cuda_stream), self._partial_ptrs, self._flag_ptrs, self._out_ptrs, self.rank, self.world,
                self.M * self.N, ctypes.c_void_p(self.state.data_ptr()), limit_ms)
            if rc != 0:
                raise RuntimeError("spmm_b200_allreduce_partials_f32_two_phase failed with cudaError %d" % rc)
        elif not self.fused:
            reduce = self._api.LIB.spmm_b200_allreduce_partials_f32_announced if self.announce \
                else self._api.LIB.spmm_b200_allreduce_partials_f32
            rc = reduce(
                ctypes.c_void_p(stream.cuda_stream), self._partial_ptrs, self._flag_ptrs, self.rank, self.world,
                ctypes.c_void_p(self.C.data_ptr()), self.M * self.N, ctypes.c_void_p(self.state.data_ptr()), limit_ms)
            if rc != 0:
                raise RuntimeError("spmm_b200_allreduce_partials_f32 failed with cudaError %d" % rc)
        return self.C
