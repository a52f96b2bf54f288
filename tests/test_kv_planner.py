"""Host-side state machines: block allocator / paged KV bookkeeping, batch layout, planner arithmetic."""
import pytest
import torch

from flyingfish_b200.config import Settings, named_shape
from flyingfish_b200.engine.batch import BatchLayout, ForwardBatch
from flyingfish_b200.engine.kv_cache import BlockAllocator, OutOfBlocks, PagedKVCache
from flyingfish_b200.planner.plan import DeviceInfo, PlanError, largest_pow2_multiple, plan_memory, workspace_row_bytes


def test_allocator_refcounts():
    a = BlockAllocator(4)
    b0, b1 = a.alloc(), a.alloc()
    assert a.free_blocks == 2
    a.share(b0)
    a.release(b0)
    assert a.free_blocks == 2
    a.release(b0)
    assert a.free_blocks == 3
    with pytest.raises(AssertionError):
        a.release(b0)
    a.alloc(); a.alloc(); a.alloc()
    with pytest.raises(OutOfBlocks):
        a.alloc()
    assert a.refcount(b1) == 1


def test_paged_reserve_commit_truncate_fork():
    kv = PagedKVCache(1, 1, 8, num_blocks=6, block_size=4, dtype=torch.float32)
    kv.add_sequence(0)
    slots = kv.reserve(0, 6)
    assert len(slots) == 6 and len(kv.seqs[0].blocks) == 2
    kv.commit(0, 6)
    # next token lands in the same second block
    s = kv.reserve(0, 1)
    assert s[0] == kv.seqs[0].blocks[1] * 4 + 2
    kv.commit(0, 2)
    kv.fork_prefix(0, 1, 4)
    assert kv.alloc.refcount(kv.seqs[0].blocks[0]) == 2
    kv.truncate(0, 3)            # speculative rollback frees the tail block
    assert len(kv.seqs[0].blocks) == 1
    kv.free_sequence(0)
    assert kv.alloc.refcount(kv.seqs[1].blocks[0]) == 1
    kv.free_sequence(1)
    assert kv.alloc.free_blocks == 6
    kv.add_sequence(2)
    with pytest.raises(OutOfBlocks):
        kv.reserve(2, 25)


def test_batch_layout_roundtrip():
    fb = ForwardBatch(BatchLayout(4, 16, 3), "cpu")
    fb.fill(ids=[5, 6, 7], positions=[0, 1, 9], slots=[64, 65, 3], q_lens=[2, 1], ctx_lens=[2, 10],
            block_rows=[[1], [0, 2]], logit_rows=[1, 2], is_decode=False, tree_mask=[1, 3, 1 << 40])
    fb.upload()
    assert fb.ids.tolist() == [5, 6, 7] and fb.q_start.tolist() == [0, 2]
    assert fb.block_table.tolist() == [[1, 0, 0], [0, 2, 0]]
    assert fb.tree_mask.tolist() == [1, 3, 1 << 40]
    assert fb.max_q_len == 2 and fb.max_ctx == 10


def test_pow2_multiple():
    assert largest_pow2_multiple(63, 64) == 0
    assert largest_pow2_multiple(64, 64) == 64
    assert largest_pow2_multiple(1000, 64) == 512
    assert largest_pow2_multiple(8192, 64) == 8192


def test_plan_memory_b200_llama8b():
    spec = named_shape("llama3-8b-shape")
    info = DeviceInfo(name="B200", sms=148, total_bytes=180 << 30, free_bytes=178 << 30)
    st = Settings(capacity=2048, max_batch=64)
    plan = plan_memory(spec, st, info, weights_bytes=16 << 30)
    assert plan.prefill_chunk % 64 == 0 and plan.prefill_chunk >= 4096
    assert plan.kv_blocks >= 32 * 64           # every sequence of the batch fits
    assert plan.kv_bytes + plan.workspace_bytes + plan.weights_bytes + plan.reserve_bytes <= info.total_bytes
    assert plan.reserve_bytes == info.total_bytes // 16
    assert workspace_row_bytes(spec) > 0


def test_plan_memory_refuses_when_too_small():
    spec = named_shape("llama3-70b-shape")
    info = DeviceInfo(name="small", total_bytes=24 << 30, free_bytes=24 << 30)
    with pytest.raises(PlanError):
        plan_memory(spec, Settings(), info, weights_bytes=140 << 30)
    # budget flag tightens the plan
    spec8 = named_shape("llama3-8b-shape")
    big = DeviceInfo(name="B200", total_bytes=180 << 30, free_bytes=178 << 30)
    p_full = plan_memory(spec8, Settings(capacity=4096, max_batch=256), big, 16 << 30)
    p_small = plan_memory(spec8, Settings(capacity=4096, max_batch=256, device_budget_gib=40), big, 16 << 30)
    assert p_small.kv_blocks < p_full.kv_blocks
