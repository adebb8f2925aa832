"""Context-parallel decode on two GPUs: sharding the KV sequence over ranks, exchanging the partials (one NCCL
all-gather, or the library's own peer stores) and merging them gives the single-GPU result. Skipped when fewer than
two GPUs are visible."""

import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, os.path.join(ROOT, "flash-sparse-attention_b200"))
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import flash_sparse_attn as fsa
    from flash_sparse_attn.ops.triton import context_parallel as cp
    from flash_sparse_attn.ops.triton.flash_dec import attn_decode

    g = torch.Generator().manual_seed(0)
    b, sk, hq, hkv, d, topk = 4, 4096, 16, 2, 128, 512
    q = torch.randn(b, hq, d, generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16).to(dev)
    idx = torch.stack([torch.randperm(sk, generator=g)[:topk] for _ in range(b)]).to(torch.int32).to(dev)
    idx[:, 5::19] = -1
    lo, hi = cp.shard_bounds(sk, world, rank)
    out, lse = cp.flash_sparse_attn_with_kvcache_cp(q, k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(), lo, hi,
                                                    gather_kv_indices=idx, softmax_threshold=-128.0, num_splits=2)
    ref, ref_lse = attn_decode("sparse", q, k, v, gather_kv_indices=idx, softmax_threshold=-128.0, num_splits=1)
    # full-context (no gather) sharding too
    out2, _ = cp.flash_sparse_attn_with_kvcache_cp(q, k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(), lo, hi,
                                                   kind="dense", num_splits=1)
    ref2, _ = attn_decode("dense", q, k, v, num_splits=1)
    # threshold on, peaked queries (tiles are skipped): every shard normalises the threshold by the whole length
    qp = (k[:, -1].repeat_interleave(hq // hkv, dim=1).float() * 3).to(torch.bfloat16)
    used = torch.full((b,), sk, dtype=torch.int32, device=dev)
    out3, _ = cp.flash_sparse_attn_with_kvcache_cp(qp, k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(), lo, hi,
                                                   gather_kv_indices=idx, softmax_threshold=1.0, num_splits=1,
                                                   seqused_k_global=used)
    ref3, _ = attn_decode("sparse", qp, k, v, gather_kv_indices=idx, softmax_threshold=-128.0, num_splits=1)
    used_local = torch.full((b,), hi - lo, dtype=torch.int32, device=dev)
    out4, _ = cp.flash_sparse_attn_with_kvcache_cp(qp, k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(), lo, hi,
                                                   softmax_threshold=1.0, num_splits=1, seqused_k_global=used,
                                                   seqused_k_local=used_local)
    ref4, _ = attn_decode("sparse", qp, k, v, softmax_threshold=-128.0, num_splits=1)
    # the same exchange through peer stores (no collective library): several steps in a row, eagerly and as a
    # replayed CUDA graph (the step counter and the buffer in use live on the device)
    # ("fused": the decode kernel stores into the peers' buffers itself; "peer": a separate push kernel)
    kl, vl = k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous()
    peer_ok = True
    for mode in ("peer", "fused"):
        dec = cp.ContextParallelDecoder(b, hq, d, torch.bfloat16, dev, num_splits=2, exchange=mode)
        for step in range(3):
            o5, l5 = dec(q, kl, vl, lo, hi, gather_kv_indices=idx, seqused_k_global=used, softmax_threshold=-128.0)
            torch.cuda.synchronize()
            peer_ok = peer_ok and (o5.float() - ref.float()).abs().max().item() < 1e-2 and \
                (l5 - ref_lse).abs().max().item() < 1e-3
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            dec(q, kl, vl, lo, hi, gather_kv_indices=idx, seqused_k_global=used, softmax_threshold=-128.0)
        for step in range(3):
            dec.out.zero_()
            graph.replay()
            torch.cuda.synchronize()
            peer_ok = peer_ok and (dec.out.float() - ref.float()).abs().max().item() < 1e-2
        torch.cuda.synchronize()
        fsa.check_status()
        dist.barrier()
        dec.peers.close()
        del graph
    close = lambda a, r: bool(((a.float() - r.float()).abs() <= 2e-2 + 2e-2 * r.float().abs()).all())  # noqa: E731
    ok = ((out.float() - ref.float()).abs().max().item() < 1e-2 and (lse - ref_lse).abs().max().item() < 1e-3
          and (out2.float() - ref2.float()).abs().max().item() < 1e-2 and close(out3, ref3) and close(out4, ref4)
          and peer_ok)
    ret[rank] = bool(ok)
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_context_parallel_decode_two_gpus():
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29700 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret.get(0) is True and ret.get(1) is True
