"""The one-shot peer-memory all-reduce fused with the residual add and the RMS norm, on ONE GPU.

The buffers of all ranks are allocated by this process on the same device and the test plays the
peers' part by hand: it writes their partials, epoch attached, into the receive regions of the
rank under test BEFORE its kernel is launched (two kernels that wait on each other are never run
side by side on one GPU).  The bounded wait is exercised with words that nothing writes."""
import pytest
import torch

from qfactory import _native
from qfactory.comm import PeerComm

pytestmark = pytest.mark.gpu


def _reference(parts, x, w, eps=1e-5):
    """Sum in rank order in fp32, rounded to fp16; x + s as one fp16 addition; the norm as rmsnorm does."""
    s = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:
        s = s + p.float()
    row = s.half() if x is None else (x + s.half())
    if w is None:
        return row, row
    f = row.float()
    n = (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + eps)).half() * w
    return row, n


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("rows,d", [(1, 8192), (5, 1024), (64, 512), (3, 16384)])
def test_allreduce_add_rmsnorm_matches_reference_over_two_calls(world, rows, d):
    g = torch.Generator(device="cuda").manual_seed(world * 100 + rows)
    rank = world - 1 if rows % 2 else 0
    comm = PeerComm.local_emulation(rank, world, d, 64)
    try:
        x = torch.randn(rows, d, generator=g, device="cuda").half()
        w = (torch.rand(d, generator=g, device="cuda") + 0.5).half()
        for call, slot in enumerate((0, 1, 0)):
            parts = [torch.randn(rows, d, generator=g, device="cuda").half() for _ in range(world)]
            assert comm.next_epoch() == call + 1
            for r in range(world):
                if r == rank:
                    comm.slot(slot, rows).copy_(parts[r])          # what the row-parallel linear writes
                else:
                    comm.write_peer_partial(r, slot, parts[r])     # what peer r's reduction kernel stores here
            want_x, want_h = _reference(parts, x, w)
            h = comm.allreduce_add_rmsnorm(slot, x, w, rows)
            torch.cuda.synchronize()
            assert torch.equal(x, want_x)                          # the residual stream, bit for bit
            assert (h.float() - want_h.float()).abs().max() <= 2e-3 * want_h.float().abs().max()
            assert comm.read_status() == 0
    finally:
        comm.close()


def test_plain_sum_without_residual_or_norm():
    world, rows, d = 4, 7, 2048
    g = torch.Generator(device="cuda").manual_seed(3)
    comm = PeerComm.local_emulation(1, world, d, 16)
    try:
        parts = [torch.randn(rows, d, generator=g, device="cuda").half() for _ in range(world)]
        for r in range(world):
            if r == 1:
                comm.slot(0, rows).copy_(parts[r])
            else:
                comm.write_peer_partial(r, 0, parts[r])
        out = comm.allreduce_add_rmsnorm(0, None, None, rows)
        torch.cuda.synchronize()
        assert torch.equal(out, _reference(parts, None, None)[0])
    finally:
        comm.close()


def test_bounded_wait_runs_out_and_the_next_call_is_correct():
    world, rows, d = 2, 2, 1024
    g = torch.Generator(device="cuda").manual_seed(5)
    comm = PeerComm.local_emulation(0, world, d, 8)
    try:
        comm.set_timeout_us(100)                                  # nothing writes the peer's words: give up after 100 us
        x = torch.randn(rows, d, generator=g, device="cuda").half()
        w = torch.ones(d, dtype=torch.float16, device="cuda")
        comm.allreduce_add_rmsnorm(0, x.clone(), w, rows)
        torch.cuda.synchronize()                                  # the kernel returned by itself
        assert comm.read_status() == 8                            # QFB_ERR_DEVICE_FLAG, reported once
        assert comm.read_status() == 0
        # the communicator is still usable: the next reduction (epoch 2, the other slot) is exact
        parts = [torch.randn(rows, d, generator=g, device="cuda").half() for _ in range(world)]
        assert comm.next_epoch() == 2
        comm.slot(1, rows).copy_(parts[0])
        comm.write_peer_partial(1, 1, parts[1])
        want_x, _ = _reference(parts, x, w)
        comm.allreduce_add_rmsnorm(1, x, w, rows)
        torch.cuda.synchronize()
        assert torch.equal(x, want_x) and comm.read_status() == 0
    finally:
        comm.close()


def test_argument_checks():
    L = _native.lib()
    comm = PeerComm.local_emulation(0, 2, 512, 4)
    try:
        x = torch.zeros(4, 512, dtype=torch.float16, device="cuda")
        call = lambda slot, rows, d: L.qfb_allreduce_add_rmsnorm(comm._h, slot, x.data_ptr(), None, None, rows, d, 1e-5, None)
        assert call(2, 1, 512) == 2          # slot out of range
        assert call(0, 1, 500) == 2          # d not a multiple of 8
        assert call(0, 5, 512) == 7          # more rows than the slot holds
        assert call(0, 0, 512) == 0          # nothing to do
        assert L.qfb_comm_max_rows() == 64
    finally:
        comm.close()


# ---- the row-parallel GEMV that sends its partial while storing it ---------------------------------
@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("M,path", [(1, "plan"), (3, "single"), (5, "cluster"), (16, "workspace"), (9, "plan")])
def test_row_parallel_gemv_sends_its_partial_in_wire_format(world, M, path):
    """`qfb_linear_forward_reduce`: the partial lands in the local slot (same bits as the plain forward)
    AND, epoch attached, in this rank's receive region of every peer's buffer, through each of the
    kernel's three store paths; the collect-only reduction then gives the reference result."""
    from oracle import qf_oracle as O
    from qfactory import QLinear

    N, K, rank = 1024, 2048, 1
    L = _native.lib()
    x, q, s, z = O.make_case(M, N, K, 4, 128, False, seed=500 + M)
    layer = QLinear.init(M, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="fragment")
    xs = x.cuda()
    comm = PeerComm.local_emulation(rank, world, N, 16)
    g = torch.Generator(device="cuda").manual_seed(M)
    try:
        if path == "single":
            L.qfb_set_gemv_tuning(1, 2)
        elif path == "cluster":
            L.qfb_set_cluster_reduce(2); L.qfb_set_gemv_tuning(4, 1)
        elif path == "workspace":
            L.qfb_set_cluster_reduce(0); L.qfb_set_gemv_tuning(4, 1)
        want = layer(xs).clone()
        resid = torch.randn(M, N, generator=g, device="cuda").half()
        w = (torch.rand(N, generator=g, device="cuda") + 0.5).half()
        for call, slot in enumerate((0, 1, 0)):
            ep = comm.next_epoch()
            assert comm.linear_into_slot(layer, xs, slot, M) is True
            torch.cuda.synchronize()
            assert _native.last_launch()["kernel"] == 3
            assert torch.equal(comm.slot(slot, M), want)
            for r in range(world):
                if r == rank:
                    continue
                words = comm.peer_words(r, slot, rank, M)
                assert torch.equal(words[:, 0::2], want.view(torch.int32))
                assert bool((words[:, 1::2] == ep).all())
            parts = [want if r == rank else torch.randn(M, N, generator=g, device="cuda").half() for r in range(world)]
            for r in range(world):
                if r != rank:
                    comm.write_peer_partial(r, slot, parts[r])
            want_x, want_h = _reference(parts, resid, w)
            h = comm.allreduce_add_rmsnorm(slot, resid, w, M, pushed=True)
            torch.cuda.synchronize()
            assert torch.equal(resid, want_x)
            assert (h.float() - want_h.float()).abs().max() <= 2e-3 * want_h.float().abs().max()
            assert comm.read_status() == 0
    finally:
        L.qfb_set_gemv_tuning(0, 0)
        L.qfb_set_cluster_reduce(1)
        comm.close()


def test_fused_activation_row_parallel_gemv_sends_its_partial():
    from qfactory import QLinear

    M, N, K, rank, world = 2, 512, 1024, 0, 4
    layer = QLinear.empty(M, K, N, 4, 128, sym=False, device="cuda", layout="fragment")
    layer.w.random_(-128, 127); layer.s.uniform_(0.002, 0.02); layer.z.view(torch.uint8).random_(0, 15)
    gu = torch.randn(M, 2 * K, device="cuda").half()
    want = layer.forward_silu_mul(gu).clone()
    comm = PeerComm.local_emulation(rank, world, N, 16)
    try:
        ep = comm.next_epoch()
        assert comm.linear_into_slot(layer, gu, 1, M, silu_mul=True) is True
        torch.cuda.synchronize()
        assert torch.equal(comm.slot(1, M), want)
        for r in range(1, world):
            words = comm.peer_words(r, 1, rank, M)
            assert torch.equal(words[:, 0::2], want.view(torch.int32)) and bool((words[:, 1::2] == ep).all())
    finally:
        comm.close()


def test_layers_the_sending_gemv_does_not_serve_fall_back_to_two_steps():
    from qfactory import QLinear

    M, N, K = 2, 512, 1024
    layer = QLinear.empty(M, K, N, 4, 128, sym=False, device="cuda", layout="tile")   # tile layout: not served
    layer.w.random_(-128, 127); layer.s.uniform_(0.002, 0.02); layer.z.view(torch.uint8).random_(0, 15)
    x = torch.randn(M, K, device="cuda").half()
    want = layer(x).clone()
    comm = PeerComm.local_emulation(0, 2, N, 16)
    try:
        assert comm.linear_into_slot(layer, x, 0, M) is False
        torch.cuda.synchronize()
        assert torch.equal(comm.slot(0, M), want)
    finally:
        comm.close()


# ---- step numbering: the receiving side inside the GEMV that consumes the sum ------------------------
def _sum_ref(parts):
    s = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:
        s = s + p.float()
    return s.half()


@pytest.mark.parametrize("world,rank", [(2, 0), (4, 3), (8, 5)])
@pytest.mark.parametrize("M", [1, 4, 16])
def test_gemv_collects_the_partials_adds_and_norms_while_staging(world, rank, M):
    """`qfb_linear_collect_addnorm_forward`: own partial from the slot, the peers' from the words they sent
    (written by hand here) for reduction idx of the current step; the new residual stream is bit-identical to
    sum-in-rank-order + one fp16 add, the output agrees with norm-then-linear within one rounding."""
    from oracle import qf_oracle as O
    from qfactory import QLinear

    N, K = 640, 2048
    x, q, s, z = O.make_case(M, N, K, 4, 128, False, seed=900 + M + world)
    layer = QLinear.init(M, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="fragment")
    comm = PeerComm.local_emulation(rank, world, K, 16)
    g = torch.Generator(device="cuda").manual_seed(world * 10 + M)
    try:
        resid = x.cuda()
        w = (torch.rand(K, generator=g, device="cuda") + 0.5).half()
        for step in range(2):
            comm.step_begin()
            for idx, slot in ((4, 0), (5, 1), (250, 0)):
                assert comm.collect_supported(layer, layer, M) in (True, False)
                ep = comm.step_epoch(idx)
                parts = [torch.randn(M, K, generator=g, device="cuda").half() for _ in range(world)]
                comm.slot(slot, M).copy_(parts[rank])
                for r in range(world):
                    if r != rank:
                        comm.write_peer_partial(r, slot, parts[r], epoch=ep)
                x_out = torch.full_like(resid, float("nan"))
                y = comm.collect_norm_linear(layer, slot, idx, resid, x_out, w, M)
                torch.cuda.synchronize()
                want_x = resid + _sum_ref(parts)
                assert torch.equal(x_out, want_x)
                f = want_x.float()
                h = (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + 1e-5)).half() * w
                y_ref = layer(h)
                assert float((y.float() - y_ref.float()).abs().max()) <= 3e-3 * float(y_ref.float().abs().max())
                assert comm.read_status() == 0
                resid = want_x
    finally:
        comm.close()


def test_step_numbered_sender_and_reduction_kernel():
    """The sending GEMV stamps reduction idx of the current step; the collecting reduction kernel accepts
    exactly that epoch and advances nothing."""
    from oracle import qf_oracle as O
    from qfactory import QLinear

    M, N, K, rank, world = 3, 1024, 2048, 1, 4
    x, q, s, z = O.make_case(M, N, K, 4, 128, False, seed=77)
    layer = QLinear.init(M, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="fragment")
    xs = x.cuda()
    want = layer(xs).clone()
    comm = PeerComm.local_emulation(rank, world, N, 16)
    g = torch.Generator(device="cuda").manual_seed(1)
    try:
        before = comm.next_epoch()
        comm.step_begin()
        for idx, slot in ((0, 0), (1, 1), (2, 0)):
            ep = comm.step_epoch(idx)
            assert comm.linear_into_slot(layer, xs, slot, M, idx=idx) is True
            torch.cuda.synchronize()
            for r in range(world):
                if r != rank:
                    words = comm.peer_words(r, slot, rank, M)
                    assert torch.equal(words[:, 0::2], want.view(torch.int32))
                    assert bool(((words[:, 1::2].to(torch.int64) & 0xFFFFFFFF) == ep).all())
            parts = [want if r == rank else torch.randn(M, N, generator=g, device="cuda").half() for r in range(world)]
            for r in range(world):
                if r != rank:
                    comm.write_peer_partial(r, slot, parts[r], epoch=ep)
            resid = torch.randn(M, N, generator=g, device="cuda").half()
            w = (torch.rand(N, generator=g, device="cuda") + 0.5).half()
            want_x, want_h = _reference(parts, resid, w)
            h = comm.allreduce_add_rmsnorm(slot, resid, w, M, idx=idx)
            torch.cuda.synchronize()
            assert torch.equal(resid, want_x)
            assert (h.float() - want_h.float()).abs().max() <= 2e-3 * want_h.float().abs().max()
        assert comm.next_epoch() == before and comm.read_status() == 0     # the per-row epochs did not move
    finally:
        comm.close()


def test_collecting_gemv_gives_up_on_words_that_never_come():
    from oracle import qf_oracle as O
    from qfactory import QLinear

    M, N, K = 2, 256, 1024
    x, q, s, z = O.make_case(M, N, K, 4, 128, False, seed=5)
    layer = QLinear.init(M, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="fragment")
    comm = PeerComm.local_emulation(0, 2, K, 8)
    try:
        comm.set_timeout_us(100)                                  # nothing writes the peer's words
        comm.step_begin()
        w = torch.ones(K, dtype=torch.float16, device="cuda")
        comm.slot(0, M).zero_()
        comm.collect_norm_linear(layer, 0, 0, x.cuda(), None, w, M)
        torch.cuda.synchronize()                                  # the launch ended by itself
        assert comm.read_status() == 8                            # QFB_ERR_DEVICE_FLAG
        ep = comm.step_epoch(1)
        part = torch.randn(M, K, device="cuda").half()
        comm.slot(1, M).copy_(part)
        comm.write_peer_partial(1, 1, part, epoch=ep)
        x_out = torch.empty(M, K, dtype=torch.float16, device="cuda")
        comm.collect_norm_linear(layer, 1, 1, x.cuda(), x_out, w, M)
        torch.cuda.synchronize()
        assert torch.equal(x_out, x.cuda() + (part.float() * 2).half()) and comm.read_status() == 0
    finally:
        comm.close()
