"""All-gather -> GEMM kernel on one GPU: the test stands in for the other ranks (their rows and flags are written into
this rank's workspace before the launch, so the kernel never waits for another kernel), and checks the product, the
rows this rank pushed into the stand-in workspaces, the flags it raised there and the epoch word."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SYMM_BYTES = 64 << 20


def _run(world, rank, rows, N, K, act, dtype, calls=2):
    from onnxruntime_b200.ops import _kernels as Kn
    dev = "cuda"
    torch.manual_seed(rank * 100 + rows)
    ws = [torch.zeros(SYMM_BYTES, dtype=torch.uint8, device=dev) for _ in range(world)]
    peers = [w.data_ptr() for w in ws]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    wt = (torch.randn(N, K, device=dev) * 0.05).to(dtype)
    bias = torch.randn(N, device=dev).to(dtype)
    assert Kn.allgather_gemm_max_rows(world, K, SYMM_BYTES) >= rows
    for call in range(1, calls + 1):          # the call's epoch; its parity picks the gather area
        shards = [(torch.randn(rows, K, device=dev) * 0.5).to(dtype) for _ in range(world)]
        shard_bytes = rows * K * 2
        for src in range(world):
            if src == rank:
                continue
            area, flag = Kn.allgather_gemm_offsets(SYMM_BYTES, call & 1, src)
            ws[rank][area + src * shard_bytes: area + (src + 1) * shard_bytes] = shards[src].view(torch.uint8).flatten()
            ws[rank][flag: flag + 4] = torch.tensor([2 * call + 1], dtype=torch.int32, device=dev).view(torch.uint8)
        out = Kn.allgather_gemm(shards[rank], wt, peers, rank, SYMM_BYTES, bias=bias, act=act, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        ref = torch.cat(shards).float() @ wt.float().t() + bias.float()
        if act == "gelu":
            ref = torch.nn.functional.gelu(ref)
        elif act == "relu":
            ref = torch.relu(ref)
        err = float((out.float() - ref).abs().max() / ref.abs().max())
        assert err < 2e-2, (call, err)
        assert int(ws[rank][64:68].view(torch.int32).item()) == call          # epoch closed
        assert int(ws[rank][68:72].view(torch.int32).item()) == 0 and int(ws[rank][76:108].view(torch.int32).abs().sum().item()) == 0
        for dst in range(world):
            if dst == rank:
                continue
            area, flag = Kn.allgather_gemm_offsets(SYMM_BYTES, call & 1, rank)
            got = ws[dst][area + rank * shard_bytes: area + (rank + 1) * shard_bytes]
            assert torch.equal(got, shards[rank].view(torch.uint8).flatten()), (call, dst)
            assert int(ws[dst][flag: flag + 4].view(torch.int32).item()) == 2 * call + 1


@pytest.mark.parametrize("world,rank,rows,N,K,act,dtype", [
    (1, 0, 128, 128, 64, "none", torch.bfloat16),
    (2, 0, 96, 384, 512, "none", torch.bfloat16),       # ragged shard: the last token tile of a shard is cut at its end
    (2, 1, 200, 200, 264, "gelu", torch.float16),       # ragged everything
    (4, 2, 320, 256, 1024, "none", torch.bfloat16),     # 256-token tiles, two per shard, second one ragged
    (8, 5, 256, 1280, 512, "none", torch.bfloat16),     # more tiles than CTAs; 256 x 256 CTA tiles
    (2, 1, 512, 640, 256, "none", torch.bfloat16),      # 256 x 256 CTA tiles, weight rows ragged
    (2, 0, 256, 128, 512, "relu", torch.float16),       # 128 x 256 CTA tiles
])
def test_allgather_gemm_with_stand_in_peers(world, rank, rows, N, K, act, dtype):
    _run(world, rank, rows, N, K, act, dtype)
