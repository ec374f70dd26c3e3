"""Tensor parallelism on real GPUs: child processes, one per GPU (needs >= 2 B200s), plus single-GPU
checks of the sharding math and of the bounded wait inside the fused all-reduce kernel."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_row_parallel_shards_sum_to_the_full_linear():
    """K-sliced trellis weights: the sum of per-shard outputs equals the unsharded linear."""
    from r4dx_b200.ops import kernels as K
    from r4dx_b200.quant import trellis
    from r4dx_b200.parallel.shard import slice_trellis_cols
    tw = trellis.random_weight(256, 1024, 4, seed=2, sigma=0.05)
    x = torch.randn(3, 1024, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
    full = K.trellis_gemv(tw.to("cuda"), x.cuda()).float()
    acc = torch.zeros_like(full)
    for r in range(4):
        sh = slice_trellis_cols(tw, 4, r)
        acc += K.trellis_gemv(sh.to("cuda"), x[:, r * 256:(r + 1) * 256].contiguous().cuda()).float()
    assert torch.allclose(acc, full, atol=0.03 * full.abs().max().item())


def test_fused_allreduce_wait_runs_out_and_reports(tmp_path):
    """A peer that never answers: the kernel gives up after its bounded spin and sets the status word."""
    import ctypes
    from r4dx_b200 import native
    from r4dx_b200.ops import kernels as K
    from r4dx_b200.parallel import tp_fused  # registers the signature
    from r4dx_b200.quant import trellis
    L = native.cuda()
    dev = "cuda"
    N, Kd, world = 256, 256, 2
    tw = trellis.random_weight(N, Kd, 4, seed=1).to(dev)
    x = torch.randn(1, Kd, device=dev).to(torch.bfloat16)
    y = torch.zeros(1, N, dtype=torch.bfloat16, device=dev)
    # both "ranks" point at the same local buffer; nobody ever writes rank 1's (value, seq) pairs
    recv = torch.zeros(2 * world * 8 * N * 2, device=dev)
    seq = torch.zeros(N // 128, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    tab = (ctypes.c_void_p * world)(recv.data_ptr(), recv.data_ptr())
    rc = L.r4dxb_trellis_gemv_allreduce(tw.words.data_ptr(), tw.suh.data_ptr(), tw.svh.data_ptr(), x.data_ptr(),
                                        y.data_ptr(), None, 0, 1, N, Kd, 4, 1, tab, seq.data_ptr(), status.data_ptr(),
                                        world, 0, 2000, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()                      # returns: the wait was bounded
    assert status.item() == 101                   # "rank 1 did not answer"
    # the context is still usable
    assert torch.isfinite(K.trellis_gemv(tw, x).float()).all()


def _run_ranks(n, script, timeout=420, args=()):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29541", script, *args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_and_library_paths_agree_on_the_same_shards(world):
    """Same shards, both communicators, full logits rows compared (prefill, decode steps, window, chunked prefill,
    after recovery); 8 ranks exercise KV-head replication."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    r = _run_ranks(world, os.path.join(ROOT, "tests", "tp_worker.py"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert f"TP_OK world={world}" in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_two_ranks():
    r = _run_ranks(2, os.path.join(ROOT, "tests", "ep_worker.py"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "EP_OK" in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pipeline_prefill_and_reshard_to_tp():
    r = _run_ranks(2, os.path.join(ROOT, "tests", "pp_worker.py"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "PP_OK" in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["split", "hybrid"])
def test_loader_products_for_pipeline_flags(mode):
    """--pp 2 (layer split) and --pp 2 --tp 2 --hybrid (pipelined prefill, reshard, tensor-parallel decode) through the
    loader and the leader/follower facade, against the whole model on one GPU."""
    r = _run_ranks(2, os.path.join(ROOT, "tests", "pp_product_worker.py"), args=(mode,))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert f"PP_PRODUCT_OK {mode}" in r.stdout
