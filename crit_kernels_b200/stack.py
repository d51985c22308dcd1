"""Column-sharded NVFP4 projection stack: the multi-GPU form of the decode GEMV.

Each projection's output columns (rows of the [N][K] weight matrix) are split evenly over the ranks of one node: rank r
holds rows [r*N/P, (r+1)*N/P) of codes, block scales and inverse scales (contiguous slices, no repacking), multiplies
the full activations by its slice, and an all-gather over NVLink assembles the [M][N] result on every rank: either
fused into the GEMV kernel's epilogue (gather="fused": every rank's gathered buffer lives in symmetric memory, the
kernel stores its results straight into all of them over NVLink and ends when every rank's results have landed here)
or as one NCCL all_gather_into_tensor after each GEMV (gather="nccl", the baseline). The K
dimension is never split: a row's sum is computed by one GPU in the order it has on a single GPU, so the gathered
output is bit-identical to the unsharded one (tests/test_stack_*.py).

The reference has no multi-GPU code; this module is new work on top of the op surface it defines.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import get_kernel


@dataclass
class Projection:
    role: str
    k: int
    n: int                      # full output width
    codes: torch.Tensor         # [n/P][k/2] uint8, this rank's rows
    scales: torch.Tensor        # [n/P][k/16] E4M3 bytes
    inverse: torch.Tensor       # [n/P] FP32


def random_nvfp4(n, k, device, generator):
    """A full NVFP4 matrix in the benchmark distribution: uniform E2M1 codes, E4M3 block scales nearest 2^u with
    u ~ U(-4, 2), global scale 1."""
    codes = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=device, generator=generator)
    scales = torch.exp2(torch.rand(n, k // 16, device=device, generator=generator) * 6 - 4).to(torch.float8_e4m3fn)
    return codes, scales.view(torch.uint8), torch.ones(n, device=device)


class FusedGatherBuffers:
    """Symmetric memory for one StackRun: every role's gathered buffer [P][M][N/P] and the pair of arrival counters,
    in one arena allocated with torch's symmetric-memory allocator and mapped into every rank's address space."""

    def __init__(self, stack, m):
        import torch.distributed._symmetric_memory as symm
        world = stack.world
        offsets, total = {}, 256                       # the counters live in the first 256 bytes
        for role, _, n in stack.roles:
            offsets[role] = total
            total += (world * m * (n // world) * 2 + 255) // 256 * 256
        self.arena = symm.empty(total, dtype=torch.uint8, device=stack.device)
        self.arena.zero_()
        self.handle = symm.rendezvous(self.arena, stack.group if stack.group is not None else dist.group.WORLD)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        array = ctypes.c_void_p * world
        self.flag_ptrs = array(*ptrs)
        self.out_ptrs = {role: array(*[p + off for p in ptrs]) for role, off in offsets.items()}
        self.full = {role: self.arena[off:off + world * m * (n // world) * 2].view(torch.bfloat16)
                     .view(world, m, n // world) for (role, _, n), off in zip(stack.roles, offsets.values())}
        torch.cuda.synchronize()
        dist.barrier(group=stack.group)                # every rank's counters are zero before anyone signals


class StackRun:
    """One captured pass over the stack at a fixed row count M."""

    def __init__(self, stack, m):
        self.stack, self.m = stack, m
        dev = stack.device
        # the first m rows of one seeded 16-row batch per role, so that row i is the same activation at every m and
        # the row-count invariance of the outputs can be checked across passes
        g = torch.Generator().manual_seed(4242)
        pin = (lambda t: t.pin_memory()) if dev.type == "cuda" else (lambda t: t)
        self.x_host = {role: pin(torch.randn(16, k, generator=g).to(torch.bfloat16)[:m].contiguous())
                       for role, k, _ in stack.roles}
        self.x = {role: t.to(dev) for role, t in self.x_host.items()}
        self.shard = {role: torch.empty(m, n // stack.world, dtype=torch.bfloat16, device=dev)
                      for role, _, n in stack.roles}
        # Gathered buffers. A rank that has finished pass k starts storing pass k + 1 (its first layers' outputs) into
        # its peers' buffers at once, while a peer may still be reading what pass k gathered (a copy to the host, a
        # comparison): see the reuse rule in include/decode_gemv_b200.h. Passes therefore alternate between two sets
        # of buffers: pass k + 2 cannot start anywhere before every rank has enqueued all of pass k + 1, which each
        # rank does after its reads of pass k.
        fused = stack.world > 1 and stack.gather.startswith("fused")
        sets = 2 if fused else 1
        self.fused_sets = [FusedGatherBuffers(stack, m) for _ in range(sets)] if fused else []
        self.passes = 0                     # passes enqueued (eager or captured): picks the set of the next one
        self.calls = 0
        self.pending = [[0, 0] for _ in range(max(sets, 1))]
        self.plain_full = None if fused else {
            role: torch.empty(stack.world, m, n // stack.world, dtype=torch.bfloat16, device=dev)
            for role, _, n in stack.roles}
        self.out_host = {role: pin(torch.empty(stack.world, m, n // stack.world, dtype=torch.bfloat16))
                         for role, _, n in stack.roles}
        self.h2d_bytes = sum(t.numel() * 2 for t in self.x_host.values())
        self.d2h_bytes = sum(t.numel() * 2 for t in self.out_host.values())
        self.kernel_launches = (len(stack.projections) if stack.batch <= 0
                                else -(-len(stack.projections) // stack.batch))
        self.graphs = []
        self.replays = 0
        self.gate_up_f32 = None
        self.batches = self._encode_batches() if stack.batch > 0 and dev.type == "cuda" else None

    def _encode_batches(self):
        """Per set of gathered buffers, the pass as launches of `stack.batch` GEMVs each (dg_encode_nvfp4_batch): a
        list of (host blob, device blob) pairs; the blobs and the pointer arrays they were made from stay alive
        here."""
        from . import cabi
        lib, st = cabi.load(), self.stack
        previous = lib.dg_set_static_weights(1 if st.static_weights else 0)     # read when a batch is encoded
        try:
            per_set = []
            for fused in (self.fused_sets or [None]):
                launches = []
                for first in range(0, len(st.projections), st.batch):
                    group = st.projections[first:first + st.batch]
                    items = (cabi.Nvfp4BatchItem * len(group))()
                    for item, p in zip(items, group):
                        x = self.x[p.role]
                        item.x, item.ldx = x.data_ptr(), x.stride(0)
                        item.codes, item.scales, item.inverse = p.codes.data_ptr(), p.scales.data_ptr(), p.inverse.data_ptr()
                        item.blocked, item.N, item.K = 0, p.codes.shape[0], p.k
                        if fused:
                            item.peer_out = ctypes.cast(fused.out_ptrs[p.role], ctypes.POINTER(ctypes.c_void_p))
                        else:
                            item.out, item.ldo = self.shard[p.role].data_ptr(), self.shard[p.role].stride(0)
                    nbytes = lib.dg_batch_blob_bytes(len(group))
                    host = torch.zeros(nbytes, dtype=torch.uint8)
                    device = torch.zeros(nbytes, dtype=torch.uint8, device=st.device)
                    code = lib.dg_encode_nvfp4_batch(
                        ctypes.cast(items, ctypes.c_void_p), len(group), 1, 1, self.m, st.world if fused else 0, st.rank,
                        fused.flag_ptrs if fused else None, (first // st.batch) & 1, ctypes.c_void_p(device.data_ptr()),
                        ctypes.c_void_p(host.data_ptr()))
                    if code:
                        raise RuntimeError(f"dg_encode_nvfp4_batch: cudaError {code}")
                    device.copy_(host)
                    launches.append((host, device, items))
                per_set.append(launches)
            torch.cuda.synchronize()
            return per_set
        finally:
            lib.dg_set_static_weights(previous)

    @property
    def fused(self):
        """The gathered buffers of the pass being enqueued."""
        return self.fused_sets[self.passes % len(self.fused_sets)] if self.fused_sets else None

    @property
    def full(self):
        """Every role's gathered buffer [P][M][N/P] as the last completed pass left it."""
        if not self.fused_sets:
            return self.plain_full
        return self.fused_sets[(self.passes - 1) % len(self.fused_sets)].full

    def eager(self, keep=None):
        """Runs the pass on the current stream; `keep` collects every projection's gathered [M][N] output."""
        st = self.stack
        previous = None
        if st.device.type == "cuda":       # the stack's weights are resident: scope the static-weights setting
            from . import cabi
            previous = cabi.load().dg_set_static_weights(1 if st.static_weights else 0)
        try:
            self._pass(keep)
        finally:
            if previous is not None:
                cabi.load().dg_set_static_weights(previous)
        self.passes += 1

    def _pass(self, keep):
        st = self.stack
        full = self.fused.full if self.fused else self.plain_full
        if self.batches is not None:
            from . import cabi
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            launches = self.batches[self.passes % len(self.batches)]
            for index, (host, _, _) in enumerate(launches):
                code = cabi.load().dg_enqueue_batch(ctypes.c_void_p(host.data_ptr()), stream)
                if code:
                    raise RuntimeError(f"dg_enqueue_batch: cudaError {code}")
                if keep is not None:       # a test reads the outputs of this launch's GEMVs (one layer at most)
                    for p in st.projections[index * st.batch:(index + 1) * st.batch]:
                        keep.append(full[p.role].permute(1, 0, 2).reshape(self.m, p.n).clone() if st.world > 1
                                    else self.shard[p.role].clone())
                    if st.world > 1:
                        # the next launch of a faster rank would store the next layer's rows into the buffers this
                        # rank is still reading (the reuse rule): every rank finishes reading first
                        torch.cuda.synchronize()
                        dist.barrier(group=st.group)
            return
        for p in st.projections:
            if self.fused:
                self._gemv_allgather(p, overlap=st.gather == "fused-overlap")
            elif st.swiglu and p.role == "gate_up":
                self._gate_up_to_down(p)
            else:
                st.kernel.gemv(self.x[p.role], p.codes, p.scales, p.inverse, self.shard[p.role])
                if st.world > 1:
                    st.nccl_gather(full[p.role], self.shard[p.role])
            if st.world > 1:
                if keep is not None:
                    if self.fused and st.gather == "fused-overlap":
                        self._collect()              # a test reads this projection's output now
                    keep.append(full[p.role].permute(1, 0, 2).reshape(self.m, p.n).clone())
            elif keep is not None:
                keep.append(self.shard[p.role].clone())
        if self.fused and st.gather == "fused-overlap":
            self._collect()

    def _collect(self):
        """End of an overlapped pass: wait for every rank's arrivals of the GEMVs enqueued since the last collect."""
        from . import cabi
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        base = ctypes.c_void_p(self.fused.arena.data_ptr())
        pending = self.pending[self.passes % len(self.fused_sets)]
        for slot in (0, 1):
            calls = pending[slot]
            if calls:
                code = cabi.load().dg_enqueue_gather_wait(base, slot, calls * self.stack.world, stream)
                if code:
                    raise RuntimeError(f"dg_enqueue_gather_wait: cudaError {code}")
                pending[slot] = 0

    def _gate_up_to_down(self, p):
        """gate_up on one GPU with SwiGLU behind it, writing the down projection's activations x["down"] = bf16 of the
        FP32 SwiGLU of the FP32 sums: as two launches (stack.swiglu = "unfused": the GEMV writes FP32 [M][2 I], the
        SwiGLU kernel reads it) or as one (dg_enqueue_nvfp4_gate_up_swiglu, "fused"). Same bits either way."""
        from . import cabi
        st, lib = self.stack, cabi.load()
        x, acts = self.x[p.role], self.x["down"]
        ptr = lambda t: ctypes.c_void_p(t.data_ptr())
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        inter = p.codes.shape[0] // 2
        if st.swiglu == "unfused":
            if self.gate_up_f32 is None:
                self.gate_up_f32 = torch.empty(self.m, 2 * inter, dtype=torch.float32, device=st.device)
            st.kernel.gemv(x, p.codes, p.scales, p.inverse, self.gate_up_f32)
            code = lib.dg_enqueue_swiglu(ptr(self.gate_up_f32), 2 * inter, 1, self.m, inter, ptr(acts), acts.stride(0), 0,
                                         stream)
        else:
            code = lib.dg_enqueue_nvfp4_gate_up_swiglu(ptr(x), x.stride(0), 1, ptr(p.codes), ptr(p.scales), 0,
                                                       ptr(p.inverse), ptr(acts), acts.stride(0), 1, self.m, inter, p.k,
                                                       stream)
        if code:
            raise RuntimeError(f"gate_up + SwiGLU ({st.swiglu}): cudaError {code}")

    def _gemv_allgather(self, p, overlap=False):
        """The GEMV with the all-gather in its epilogue (C ABI dg_enqueue_nvfp4_allgather) on the current stream."""
        from . import cabi
        st, x = self.stack, self.x[p.role]
        ptr = lambda t: ctypes.c_void_p(t.data_ptr())
        code = cabi.load().dg_enqueue_nvfp4_allgather(
            ptr(x), x.stride(0), 1, ptr(p.codes), ptr(p.scales), 0, ptr(p.inverse), self.fused.out_ptrs[p.role],
            self.fused.flag_ptrs, st.world, st.rank, (self.calls & 1) + (2 if overlap else 0), 1, self.m,
            p.codes.shape[0], p.k,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        if code:
            raise RuntimeError(f"dg_enqueue_nvfp4_allgather: cudaError {code}")
        if overlap:
            self.pending[self.passes % len(self.fused_sets)][self.calls & 1] += 1
        self.calls += 1

    def capture(self):
        side = torch.cuda.Stream(device=self.stack.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.eager()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        # one graph per set of gathered buffers; replays take them in turn (an even number of warm-up passes above,
        # so the first graph is captured on set 0)
        for _ in range(max(len(self.fused_sets), 1)):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.eager()
            self.graphs.append(graph)
        self.passes = 0
        return self

    def replay(self):
        self.graphs[self.replays % len(self.graphs)].replay()
        self.replays += 1
        self.passes = self.replays

    def outputs(self):
        """Every role's output [M][N] of the last completed pass (the last layer's, since layers share buffers)."""
        if self.stack.world > 1:
            return {role: self.full[role].permute(1, 0, 2).reshape(self.m, -1) for role, _, _ in self.stack.roles}
        return {role: self.shard[role] for role, _, _ in self.stack.roles}

    def replay_e2e(self):
        """A pass as a caller with host buffers sees it: activations up, the pass, every role's output down."""
        for role, host in self.x_host.items():
            self.x[role].copy_(host, non_blocking=True)
        self.replay()
        for role, _, _ in self.stack.roles:
            src = self.full[role] if self.stack.world > 1 else self.shard[role].view_as(self.out_host[role])
            self.out_host[role].copy_(src, non_blocking=True)
        torch.cuda.synchronize()


@dataclass
class ShardedStack:
    projections: list
    roles: tuple
    rank: int
    world: int
    device: torch.device
    group: object = None
    kernel: object = None
    gather: str = "fused"       # "fused": all-gather in the GEMV epilogue over symmetric memory; "nccl": NCCL per GEMV
    static_weights: bool = True
    seed: int = 0
    layers: int = 0
    swiglu: str = ""            # "unfused" / "fused" (one GPU): gate_up's SwiGLU feeds the layer's down projection
    batch: int = 0              # > 0: that many consecutive GEMVs per launch (dg_enqueue_batch), legal because the
                                # stack's GEMVs do not read each other's outputs; with gather="fused" only

    @property
    def gather_kind(self):
        if self.world == 1:
            return "none (1 GPU)"
        if self.gather == "fused" and self.batch > 0:
            return (f"fused, {self.batch} GEMVs a launch: rows stored into every rank's symmetric buffer as each GEMV "
                    "finishes, arrivals exchanged once per launch")
        if self.gather == "fused":
            return "fused into the GEMV epilogue: peer stores into every rank's symmetric buffer + arrival counters"
        if self.gather == "fused-overlap":
            return ("fused into the GEMV epilogue, arrivals collected once at the end of the pass (legal only because "
                    "the stack's GEMVs do not consume each other's outputs)")
        return "NCCL all_gather_into_tensor after every GEMV, inside the graph"

    def nccl_gather(self, full, shard):
        """full [P][M][N/P] <- every rank's shard [M][N/P]."""
        dist.all_gather_into_tensor(full.view(-1, shard.shape[1]), shard, group=self.group)

    @classmethod
    def random(cls, layers, roles, rank, world, device, seed=0, group=None, kernel=None, gather="fused",
               static_weights=True, batch=0):
        """`layers` x `roles` projections. static_weights: the stack's weights are resident and never rewritten, so
        every GEMV of a pass may start streaming them while the kernels before it finish (dg_set_static_weights is
        switched on for the duration of each enqueued pass and restored after it). Every rank draws the same full
        matrix from the same seed and keeps its rows, so the shards of all ranks together are exactly the matrix a
        single GPU would hold."""
        projections = []
        for layer in range(layers):
            for idx, (role, k, n) in enumerate(roles):
                if n % world:
                    raise ValueError(f"{role}: N={n} does not split over {world} ranks")
                g = torch.Generator(device=device).manual_seed(seed * 1000003 + layer * 16 + idx)
                codes, scales, inverse = random_nvfp4(n, k, device, g)
                lo, hi = rank * n // world, (rank + 1) * n // world
                projections.append(Projection(role, k, n, codes[lo:hi].clone(), scales[lo:hi].clone(),
                                              inverse[lo:hi].clone()))
                del codes, scales, inverse
        if gather not in ("fused", "fused-overlap", "nccl"):
            raise ValueError(f"gather must be 'fused', 'fused-overlap' or 'nccl', not {gather!r}")
        if batch > 0 and world > 1 and gather != "fused":
            raise ValueError("batched launches carry their own all-gather: gather must be 'fused'")
        return cls(projections, tuple(roles), rank, world, device, group, kernel or get_kernel(), gather,
                   static_weights, seed, layers, "", batch)

    def with_swiglu(self, mode):
        """The same shards with each layer's down projection fed by the SwiGLU of its gate_up projection, as two
        launches ("unfused") or in gate_up's epilogue ("fused")."""
        import dataclasses
        if self.world != 1 or mode not in ("unfused", "fused"):
            raise ValueError("SwiGLU between gate_up and down is wired for one GPU, mode 'unfused' or 'fused'")
        return dataclasses.replace(self, swiglu=mode)

    def with_batch(self, batch):
        """The same shards launched `batch` GEMVs at a time (0: one launch per GEMV)."""
        import dataclasses
        return dataclasses.replace(self, batch=batch)

    @staticmethod
    def full_matrix(seed, layer, idx, role_k_n, device):
        """The whole (unsharded) matrix of projection `idx` of `layer`, as every rank draws it before keeping its rows."""
        _, k, n = role_k_n
        g = torch.Generator(device=device).manual_seed(seed * 1000003 + layer * 16 + idx)
        return random_nvfp4(n, k, device, g)

    def capture(self, m):
        return StackRun(self, m).capture()

    def run(self, m):
        """Eager pass; returns every projection's gathered output (for tests)."""
        keep = []
        StackRun(self, m).eager(keep)
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        return keep
