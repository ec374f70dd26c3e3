"""The fused compute+collective kernels on ONE GPU: rank 0 of a 2-rank group against a scripted peer.

The peer's receive buffer is a second local buffer; what the peer would push is written by the test beforehand
(value, sequence) - or not written at all, to make a bounded wait run out.  No second GPU, no second kernel that
waits on this one, no fault: a wait that runs out sets a status word the host reads, and the context stays usable.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _setup(N=1024, Kd=512, seed=1):
    from r4dx_b200 import native
    from r4dx_b200.ops import kernels as K
    from r4dx_b200.parallel import tp_fused  # noqa: F401 (registers signatures)
    from r4dx_b200.quant import trellis
    dev = "cuda"
    w = trellis.random_weight(N, Kd, 4, seed=seed, device=dev)
    slot_pairs = 2 * 8 * N
    recv = [torch.zeros(2 * slot_pairs, 2, dtype=torch.float32, device=dev) for _ in range(2)]
    tab = (ctypes.c_void_p * 2)(*[r.data_ptr() for r in recv])
    return native.cuda(), K, w, recv, tab, slot_pairs


def _peer_push(recv0, slot_pairs, N, seq, value, rows=8):
    """What rank 1 stores into rank 0's buffer for call number ``seq`` (u32, may wrap)."""
    bits = torch.tensor([seq & 0xFFFFFFFF], dtype=torch.int64).to(torch.int32 if seq < 2 ** 31 else torch.int64)
    seq_f = torch.tensor([seq & 0xFFFFFFFF], dtype=torch.int64).view(torch.int32)[0:1].view(torch.float32).item()
    blk = recv0[(seq & 1) * slot_pairs + 8 * N:(seq & 1) * slot_pairs + (8 + rows) * N]
    blk[:, 0] = value
    blk[:, 1] = seq_f


def _call(L, K, w, x, res, tab, block_seq, status, spin, impl="simt"):
    if impl == "mma":
        return L.r4dxb_trellis_gemv_mma_allreduce(
            w.words.data_ptr(), w.suh.data_ptr(), w.svh.data_ptr(), x.data_ptr(), res.data_ptr(), res.data_ptr(), K.PRO_NONE,
            x.shape[0], w.N, w.K, w.kb, K.pick_ksplit(w.N, w.K), tab, block_seq.data_ptr(), status.data_ptr(), 2, 0, spin,
            K.gemm_status("cuda").data_ptr(), torch.cuda.current_stream().cuda_stream)
    return L.r4dxb_trellis_gemv_allreduce(w.words.data_ptr(), w.suh.data_ptr(), w.svh.data_ptr(), x.data_ptr(), res.data_ptr(),
                                          res.data_ptr(), K.PRO_NONE, x.shape[0], w.N, w.K, w.kb, K.pick_ksplit(w.N, w.K), tab,
                                          block_seq.data_ptr(), status.data_ptr(), 2, 0, spin, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("impl", ["simt", "mma"])
def test_scripted_peer_sum_is_rank_ordered_and_survives_sequence_wrap(impl):
    L, K, w, recv, tab, sp = _setup()
    N = w.N
    g = torch.Generator().manual_seed(0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # start just below the wrap of the 32-bit call counter: calls 0xFFFFFFFE, 0xFFFFFFFF, 0, 1
    start = 0xFFFFFFFD
    block_seq = torch.full((N // 128,), start - 2 ** 32, dtype=torch.int64).to(torch.int32).cuda()
    for i in range(4):
        seq = (start + 1 + i) & 0xFFFFFFFF
        x = torch.randn(3, w.K, generator=g).to(BF).cuda()
        res0 = torch.randn(3, N, generator=g).to(BF).cuda()
        res = res0.clone()
        _peer_push(recv[0], sp, N, seq, 0.25 * (i + 1))
        assert _call(L, K, w, x, res, tab, block_seq, status, 1 << 16, impl) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        K.check_gemm_status("cuda")
        own = K.trellis_gemv(w, x).float()
        want = (own + 0.25 * (i + 1) + res0.float())
        assert torch.allclose(res.float(), want, atol=0.03 * want.abs().max().item(), rtol=2e-2)
        # what rank 0 pushed to its peer: its own partial, stamped with the same sequence number
        mine = recv[1][(seq & 1) * sp:(seq & 1) * sp + 3 * N]
        assert torch.equal(mine[:, 1].view(torch.int32), torch.full((3 * N,), seq - (2 ** 32 if seq >= 2 ** 31 else 0), dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("impl", ["simt", "mma"])
def test_a_wait_that_runs_out_reports_the_missing_rank_and_leaves_the_context_usable(impl):
    L, K, w, recv, tab, sp = _setup(seed=2)
    N = w.N
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    block_seq = torch.zeros(N // 128, dtype=torch.int32, device="cuda")
    x = torch.randn(1, w.K).to(BF).cuda()
    res = torch.zeros(1, N, dtype=BF, device="cuda")
    assert _call(L, K, w, x, res, tab, block_seq, status, 1 << 10, impl) == 0  # nobody pushes: the wait gives up quickly
    torch.cuda.synchronize()
    assert int(status.item()) == 101                                          # 100 + the rank that never answered
    # sticky: with the word still set, the next hundred calls do not wait at all (generous limit, still quick)
    import time
    t0 = time.perf_counter()
    for _ in range(100):
        assert _call(L, K, w, x, res, tab, block_seq, status, 1 << 22, impl) == 0
    torch.cuda.synchronize()
    assert (time.perf_counter() - t0) / 100 < 1e-3
    assert int(status.item()) == 101
    assert int(block_seq[0].item()) == 101                                    # counters still advance, so a recovery can rebase them
    # the device is fine: an ordinary product right after gives the right answer
    y = K.trellis_gemv(w, x)
    from r4dx_b200.quant import trellis
    ref = x.float().cpu() @ trellis.reconstruct(trellis.TrellisWeight(w.words.cpu(), w.suh.cpu(), w.svh.cpu(), w.N, w.K, w.kb)).T
    assert torch.allclose(y.float().cpu(), ref, atol=0.03 * ref.abs().max().item(), rtol=2e-2)


def test_prefill_wait_kernel_times_out_with_its_code_and_passes_when_the_count_is_there():
    from r4dx_b200 import native
    from r4dx_b200.parallel import tp_fused  # noqa: F401
    L = native.cuda()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert L.r4dxb_tp_wait(flag.data_ptr(), 5, 1 << 8, 303, status.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 303
    status.zero_()
    flag.fill_(7)
    assert L.r4dxb_tp_wait(flag.data_ptr(), 5, 1 << 8, 303, status.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
