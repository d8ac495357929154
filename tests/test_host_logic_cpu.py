"""CPU tests of the host-side logic: registry and backend contracts (mirroring the reference's
own contract tests, capstone-project/tests/test_kernel.py:33-75, 146-177 and
tests/test_ltx_routing.py:147-190), (batch, head) sharding plans, the ring schedule, and a
world_size-2 gloo run of both multi-GPU plans with the arithmetic done by the CPU oracle."""

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from b200_attention_b200 import backend, registry, ring, sharding
from oracle import sdpa_oracle as O


# ---------------------------------------------------------------------------------- registry
def test_registry_resolves_kernels_and_shapes():
    spec = registry.resolve_kernel("b200")
    assert spec.launch_symbol == "b200attn_bhld_launch" and spec.len_q_multiple == 1
    assert registry.resolve_kernel(20).layout == "bshd"
    assert registry.resolve_kernel("b200attn_bshd_launch").op_name == "sdpa_bshd"
    with pytest.raises(ValueError):
        registry.resolve_kernel("")
    with pytest.raises(ValueError):
        registry.resolve_kernel("18")
    assert registry.resolve_shape("paper8k") == ("paper8k", 4, 16, 8192, 8192)
    with pytest.raises(ValueError):
        registry.resolve_shape("paper1k")
    assert len(registry.source_closure_sha256(spec)) == 64


def test_registry_loads_shim_and_refuses_cpu_tensors(native_built):
    module = registry.load_kernel(registry.resolve_kernel("b200"))
    x = torch.zeros(1, 2, 256, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="must be CUDA tensors"):
        module.sdpa(x, x, x)


# ----------------------------------------------------------------------------------- backend
def test_backend_constructor_is_lazy_and_mask_is_rejected_first():
    attn = backend.B200Attention()
    assert attn.label == "B200Attention" and attn._loaded is False
    # a mask is refused before any tensor or CUDA check: arbitrary objects are fine here
    with pytest.raises(RuntimeError, match="unmasked"):
        attn(object(), object(), object(), 32, mask=object())


def test_backend_rejections():
    attn = backend.B200Attention()
    x = torch.zeros(1, 256, 256, dtype=torch.bfloat16)
    with pytest.raises(TypeError):
        attn(x, x, "v", 2)
    for bad_heads in (0, -1, 2.0, True):
        with pytest.raises(ValueError):
            attn(x, x, x, bad_heads)
    with pytest.raises(RuntimeError, match="CUDA"):
        attn(x, x, x, 2)
    backend.reset_stats()
    assert backend.get_stats() == {"total_calls": 0, "signatures": {}, "unique_inputs": []}


def test_backend_hook_receives_the_exact_callable():
    # `with_attention` of the video model returns a new stage holding the callable it was given
    class FakeStage:
        def __init__(self, attention=None):
            self.attention = attention

        def with_attention(self, fn):
            return FakeStage(fn)

    attn = backend.B200Attention()
    base = FakeStage()
    routed = base.with_attention(attn)
    assert routed is not base and routed.attention is attn and base.attention is None


def test_stats_signature_format():
    q = torch.zeros(1, 512, 256, dtype=torch.bfloat16)
    k = torch.zeros(1, 128, 256, dtype=torch.bfloat16)
    backend.reset_stats()
    backend._LOG.add((q, k, k), (1, 512, 128, 2, 128))
    backend._LOG.add((q, k, k), (1, 512, 128, 2, 128))
    stats = backend.get_stats()
    assert stats["total_calls"] == 2
    assert stats["signatures"] == {"B=1,Lq=512,Lkv=128,H=2,D=128,dtype=torch.bfloat16,device=cpu": 2}
    assert len(stats["unique_inputs"]) == 1
    backend.reset_stats()


# ---------------------------------------------------------------------------------- sharding
@pytest.mark.parametrize("batch,heads,world", [(4, 16, 1), (4, 16, 2), (4, 16, 8), (1, 12, 8), (3, 5, 4), (1, 1, 4)])
def test_sharding_plan_partitions_every_unit_once(batch, heads, world):
    seen = []
    for r in range(world):
        for hr in sharding.plan(batch, heads, world, r):
            assert 0 <= hr.head_begin < hr.head_end <= heads and 0 <= hr.batch < batch
            seen += [(hr.batch, h) for h in range(hr.head_begin, hr.head_end)]
    assert sorted(seen) == [(b, h) for b in range(batch) for h in range(heads)]
    counts = [sharding.units_of(p) for p in sharding.plan_all(batch, heads, world)]
    assert max(counts) - min(counts) <= 1


def test_sharding_launches_merge_whole_batch_entries():
    assert sharding.launches_of(sharding.plan(4, 16, 1, 0), 16) == [(0, 4, 0, 16)]
    assert sharding.launches_of(sharding.plan(4, 16, 2, 1), 16) == [(2, 4, 0, 16)]
    assert sharding.launches_of(sharding.plan(4, 16, 8, 3), 16) == [(1, 2, 8, 16)]
    # 3 x 5 units over 4 ranks: rank 1 owns heads 4 of batch 0 and heads 0..2 of batch 1
    assert sharding.launches_of(sharding.plan(3, 5, 4, 1), 5) == [(0, 1, 4, 5), (1, 2, 0, 3)]
    # a rank that owns a partial range, whole entries, and a partial range again
    ranges = [sharding.HeadRange(0, 3, 5), sharding.HeadRange(1, 0, 5), sharding.HeadRange(2, 0, 5),
              sharding.HeadRange(3, 0, 2)]
    assert sharding.launches_of(ranges, 5) == [(0, 1, 3, 5), (1, 3, 0, 5), (3, 4, 0, 2)]


def test_sharding_main_config_is_even():
    for world in (1, 2, 4, 8):
        assert sharding.imbalance(4, 16, world) == 1.0
    assert sharding.flat_bounds(64, 8, 3) == (24, 32)
    with pytest.raises(ValueError):
        sharding.flat_bounds(8, 2, 2)


# -------------------------------------------------------------------------------------- ring
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ring_schedule_and_flags(world):
    for r in range(world):
        order = ring.ring_schedule(world, r)
        assert order[0] == r and sorted(order) == list(range(world))
    # at every step each shard is read by exactly one rank
    for s in range(world):
        assert sorted(ring.ring_schedule(world, r)[s] for r in range(world)) == list(range(world))
    flags = ring.chain_flags(world)
    assert flags[0][0] is False and flags[-1][1] is False
    assert all(m for m, _ in flags[1:]) and all(e for _, e in flags[:-1])
    for step in ring.pull_plan(world):
        assert sorted(o for _, o in step) == list(range(world))
        assert all(reader != owner for reader, owner in step)


# ------------------------------------------------------------------------ gloo, world size 2
def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, result_queue):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, L = 2, 3, 64
        q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(B, H, L, L, seed=40))
        full_o, full_lse = O.sdpa_explicit(q, k, v)

        # (batch, head) sharding: each rank computes its slices; all_reduce only assembles them
        out = torch.zeros_like(full_o)
        for hr in sharding.plan(B, H, world, rank):
            sl = (slice(hr.batch, hr.batch + 1), slice(hr.head_begin, hr.head_end))
            out[sl], _ = O.sdpa_explicit(q[sl], k[sl], v[sl])
        dist.all_reduce(out)
        ok_shard = bool((out - full_o).abs().max() < 1e-5)

        # sequence-parallel ring: rows of Q sharded, K/V shards visited in ring order and merged
        rows = slice(rank * L // world, (rank + 1) * L // world)
        shards = [(k[:, :, r * L // world:(r + 1) * L // world], v[:, :, r * L // world:(r + 1) * L // world])
                  for r in range(world)]
        acc = None
        for step, (merge, emit) in zip(ring.ring_schedule(world, rank), ring.chain_flags(world)):
            o_s, lse_s = O.sdpa_explicit(q[:, :, rows], *shards[step])
            acc = (o_s, lse_s) if not merge else O.merge_partials(acc[0], acc[1], o_s, lse_s)
        ok_ring = bool((acc[0] - full_o[:, :, rows]).abs().max() < 1e-5 and
                       (acc[1] - full_lse[:, :, rows]).abs().max() < 1e-5)
        flags = torch.tensor([int(ok_shard), int(ok_ring)])
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        if rank == 0:
            result_queue.put(flags.tolist())
    finally:
        dist.destroy_process_group()


def _run_ranks(target, world: int, results: int, attempts: int = 2):
    """Starts `world` ranks of `target(rank, world, port, queue)` and returns `results` queue
    entries. A rendezvous that fails (the port found free was taken in between, a rank too slow to
    start on a loaded machine) is tried once more on another port; a second failure stands."""
    for attempt in range(attempts):
        ctx = mp.get_context("spawn")
        queue = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=target, args=(r, world, port, queue)) for r in range(world)]
        for p in procs:
            p.start()
        got = []
        try:
            for _ in range(results):
                got.append(queue.get(timeout=240))
        except Exception:
            got = None
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
                p.join()
        if got is not None and all(p.exitcode == 0 for p in procs):
            return got
        if attempt + 1 == attempts:
            raise AssertionError(f"ranks failed: exit codes {[p.exitcode for p in procs]}, results {got}")


def test_two_rank_gloo_sharding_and_ring():
    assert _run_ranks(_worker, 2, results=1) == [[1, 1]]


# ------------------------------------------------- ring host failure paths, gloo, world size 2
class _FakeNative:
    """Stand-in for the ctypes binding: IPC export/open/close without a GPU. `fail_open_on` makes
    b200attn_ipc_open return a non-zero status on that rank, after `fail_after` successful opens."""

    STATUS_CUDA = 4

    class Error(RuntimeError):
        def __init__(self, status):
            super().__init__(f"status {status}")
            self.status = status

    def __init__(self, rank, fail_open_on=None, fail_after=0):
        self.rank, self.fail_open_on, self.fail_after = rank, fail_open_on, fail_after
        self.opened, self.closed = [], []

    def lib(self):
        return self

    def check(self, status):
        if status != 0:
            raise _FakeNative.Error(status)

    def b200attn_ipc_export(self, ptr, handle, off):
        import ctypes as C

        C.memmove(handle, int(ptr).to_bytes(8, "little") * 8, 64)
        off._obj.value = 0
        return 0

    def b200attn_ipc_open(self, raw, base):
        if self.fail_open_on == self.rank and len(self.opened) >= self.fail_after:
            return self.STATUS_CUDA
        value = int.from_bytes(raw[:8], "little")
        base._obj.value = value
        self.opened.append(value)
        return 0

    def b200attn_ipc_close(self, base):
        self.closed.append(base.value)
        return 0


def _ring_failure_worker(rank: int, world: int, port: int, result_queue):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    out = {}
    try:
        # 1. shards of different shapes: every rank raises, nothing stays mapped
        fake = _FakeNative(rank)
        ra = ring.RingAttention(native=fake)
        shard = torch.zeros(1, 2, 128 * (rank + 1), 128, dtype=torch.bfloat16)
        try:
            ra.bind(shard, shard.clone())
            out["mismatch"] = "no error"
        except RuntimeError as exc:
            out["mismatch"] = "differ in shape" in str(exc)
        out["mismatch_clean"] = ra._peers == [] and fake.opened == []

        # 2. the second IPC open fails on rank 1: it surfaces as the status, and what had been
        #    opened before is closed again; rank 0 binds normally and unbinds normally
        fake = _FakeNative(rank, fail_open_on=1, fail_after=1)
        ra = ring.RingAttention(native=fake)
        k, v = torch.zeros(1, 2, 128, 128, dtype=torch.bfloat16), torch.zeros(1, 2, 128, 128, dtype=torch.bfloat16)
        try:
            ra.bind(k, v)
            out["open"] = "bound"
            ra.unbind()
        except _FakeNative.Error as exc:
            out["open"] = exc.status
        out["open_clean"] = sorted(fake.opened) == sorted(fake.closed) and ra._peers == []
        out["opened"] = len(fake.opened)
    except Exception as exc:
        out["error"] = repr(exc)
    finally:
        result_queue.put((rank, out))
        dist.destroy_process_group()


def test_two_rank_gloo_ring_failure_paths():
    results = dict(_run_ranks(_ring_failure_worker, 2, results=2))
    for rank in (0, 1):
        assert "error" not in results[rank], results[rank]
        assert results[rank]["mismatch"] is True and results[rank]["mismatch_clean"], results[rank]
        assert results[rank]["open_clean"], results[rank]
    assert results[0]["open"] == "bound" and results[0]["opened"] == 2
    assert results[1]["open"] == _FakeNative.STATUS_CUDA and results[1]["opened"] == 1
