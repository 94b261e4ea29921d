"""How many cache pages the engine plans for each group of layers (no GPU: the device's memory figures are
given by the test).  The reference sizes its pool as max_num_seqs * ceil(max_model_len / 16)
(crates/rllm-server/src/server.rs:367-370); its formula from free memory is
crates/rllm-cache/src/spec.rs:45-60."""
from types import SimpleNamespace

import pytest
import torch

from rllm_b200.cache import page_bytes
from rllm_b200.config.engine_args import EngineArgs
from rllm_b200.engine import engine_core
from rllm_b200.parts.spec import KVPagesNeed, StateNeed


def fake_model(groups, owners, dtype=torch.bfloat16, hidden=64, vocab=1000):
    layout = SimpleNamespace(groups=groups, owners=owners)
    return SimpleNamespace(layout=layout, dtype=dtype, spec=SimpleNamespace(hidden_size=hidden, vocab_size=vocab))


def test_explicit_count_and_windowed_groups_take_no_more_than_they_can_use():
    full, win, state = KVPagesNeed(2, 16, None), KVPagesNeed(2, 16, 24), StateNeed((8,))
    m = fake_model([full, state, win], [[0, 2], [1], [3]])
    args = EngineArgs(num_gpu_blocks=500, block_size=16, max_num_seqs=4, max_num_batched_tokens=64,
                      long_prefill_token_threshold=32)
    # the windowed group: 4 requests x (ceil((24 + 32) / 16) + 1) = 20 pages
    assert engine_core.plan_cache_pages(m, args, 4096, torch.device("cpu")) == [500, 20]
    args.num_gpu_blocks = 7
    assert engine_core.plan_cache_pages(m, args, 4096, torch.device("cpu")) == [7, 7]


def test_counts_from_free_memory(monkeypatch):
    full, win = KVPagesNeed(8, 64, None), KVPagesNeed(8, 64, 1024)
    m = fake_model([full, win], [list(range(12)), list(range(12, 16))], hidden=2048, vocab=128256)
    args = EngineArgs(block_size=16, max_num_seqs=64, max_num_batched_tokens=2048, gpu_memory_utilization=0.5)
    GiB = 1 << 30
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device=None: (170 * GiB, 180 * GiB))
    # plenty of room: every group gets all it can use
    pages = engine_core.plan_cache_pages(m, args, 8192, torch.device("cpu"))
    assert pages == [64 * 512, 64 * ((1024 + 2048) // 16 + 1)]
    # little room: both groups shrink by the same share, and the bytes stay inside the budget
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device=None: (12 * GiB, 180 * GiB))
    args.gpu_memory_utilization = 0.97
    small = engine_core.plan_cache_pages(m, args, 8192, torch.device("cpu"))
    assert small[0] < pages[0] and abs(small[0] / pages[0] - small[1] / pages[1]) < 1e-3
    used = small[0] * page_bytes(full, 16, 2) * 12 + small[1] * page_bytes(win, 16, 2) * 4
    budget = int(180 * GiB * 0.97) - 168 * GiB
    assert 0 < used <= budget
    # no room at all
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device=None: (1 * GiB, 180 * GiB))
    with pytest.raises(RuntimeError, match="no room for a KV cache"):
        engine_core.plan_cache_pages(m, args, 8192, torch.device("cpu"))


def test_a_model_without_pages_needs_none():
    m = fake_model([StateNeed((4,))], [[0]])
    assert engine_core.plan_cache_pages(m, EngineArgs(), 128, torch.device("cpu")) == []
