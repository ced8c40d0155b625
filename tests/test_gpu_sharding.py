"""Head sharding over two GPUs with NCCL: every rank attends to its own heads, the optional all-gather
reassembles the full output.  Skipped when fewer than two GPUs are visible."""

import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, heads, seq, result):
    sys.path.insert(0, os.path.join(ROOT, "open-vc-attention_b200"))
    import torch.distributed as dist

    import open_vc_attn
    from open_vc_attn.forward import check_status
    from open_vc_attn.sharding import attention_head_sharded, head_range

    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=device)
    try:
        g = torch.Generator(device="cpu").manual_seed(5)
        q, k, v = [torch.randn(seq, heads, 128, generator=g).to(torch.bfloat16).to(device) for _ in range(3)]
        local = attention_head_sharded(q, k, v)
        full = attention_head_sharded(q, k, v, gather=True)
        check_status(device)
        h0, h1 = head_range(heads, world, rank)
        single = open_vc_attn.attention(q, k, v)
        result[rank] = bool(torch.equal(local, single[:, h0:h1]) and torch.equal(full, single))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("heads", [4, 5])
def test_two_ranks_match_one_gpu(heads):
    import torch.multiprocessing as mp

    manager = mp.Manager()
    result = manager.dict()
    ctx = mp.get_context("spawn")
    port = 29700 + (os.getpid() % 200) + heads
    procs = [ctx.Process(target=_worker, args=(r, 2, port, heads, 700, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert result[0] and result[1]
