"""Host-side logic of the serving engine: block manager and scheduler (no GPU)."""
from nanoquantization_b200.engine import BlockManager, Scheduler, Sequence


def test_block_manager_allocates_and_releases():
    bm = BlockManager(num_blocks=6, block_size=4)
    s = Sequence(0, [1] * 9, 4)
    assert bm.ensure(s, 9) and len(s.blocks) == 3 and len(bm.free) == 3
    assert bm.ensure(s, 12) and len(s.blocks) == 3          # still fits
    assert bm.ensure(s, 13) and len(s.blocks) == 4
    t = Sequence(1, [1] * 20, 1)
    assert not bm.ensure(t, 20) and t.blocks == []           # pool exhausted: nothing taken
    bm.release(s)
    assert len(bm.free) == 6 and s.blocks == []


def test_scheduler_prefill_first_then_decode_and_finish():
    bm = BlockManager(num_blocks=16, block_size=4)
    sch = Scheduler(bm, max_batch=2, max_prefill_tokens=64)
    seqs = [Sequence(i, [7] * 5, 2) for i in range(3)]
    for s in seqs:
        sch.add(s)
    kind, batch = sch.step()
    assert kind == "prefill" and [s.seq_id for s in batch] == [0, 1]      # max_batch = 2
    for s in batch:
        s.output.append(1)
    assert sch.finish_step(kind, batch) == []
    kind, batch = sch.step()
    assert kind == "decode" and len(batch) == 2                             # third waits for a free seat
    for s in batch:
        s.output.append(2)
    done = sch.finish_step(kind, batch)
    assert {s.seq_id for s in done} == {0, 1} and len(bm.free) == 16
    kind, batch = sch.step()
    assert kind == "prefill" and batch[0].seq_id == 2


def test_scheduler_preempts_when_blocks_run_out():
    bm = BlockManager(num_blocks=4, block_size=4)
    sch = Scheduler(bm, max_batch=4, max_prefill_tokens=64)
    a, b = Sequence(0, [1] * 7, 8), Sequence(1, [1] * 7, 8)
    sch.add(a); sch.add(b)
    kind, batch = sch.step()
    assert kind == "prefill" and len(batch) == 2 and len(bm.free) == 0
    for s in batch:
        s.output.append(5)
    sch.finish_step(kind, batch)
    kind, batch = sch.step()          # both need a third block, none is free: the youngest is preempted
    assert kind == "decode" and [s.seq_id for s in batch] == [0]
    assert sch.waiting[0].seq_id == 1 and sch.waiting[0].prompt == [1] * 7 + [5] and sch.waiting[0].blocks == []


def test_engine_rejects_a_prompt_the_cache_can_never_hold():
    import pytest
    import torch
    from nanoquantization_b200.engine import LLMEngine
    from nanoquantization_b200.models.qwen3_quantized import Qwen3QuantizedForCausalLM
    model = Qwen3QuantizedForCausalLM(1, 64, 128, 2, 1, 32, 128, 4, 128, 64, device="cpu", dtype=torch.float16)
    eng = LLMEngine(model, num_blocks=2, block_size=4, max_batch=2, use_cuda_graph=False)
    with pytest.raises(ValueError, match="never be admitted"):
        eng.add_request([1] * 8, 4)       # 8 prompt tokens + 1 generated > 2 blocks of 4
    assert eng.add_request([1] * 7, 1) == 0
