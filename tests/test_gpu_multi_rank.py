"""The peer-memory all-reduce between REAL ranks: one process per GPU (needs at least two GPUs on
the box; skipped otherwise), buffers exchanged as IPC handles over the NCCL process group.  Every
rank regenerates the partials of all ranks from seeds and checks the fused all-reduce + residual
add + RMS norm bit for bit (residual stream) and within an fp16 step (normed row), launched one
by one and replayed from a CUDA graph; then the tensor-parallel decoder against the unsharded one."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _partial(rank, it, rows, d, dev):
    g = torch.Generator(device=dev).manual_seed(1000 * it + rank)
    return torch.randn(rows, d, generator=g, device=dev).half()


def _expected(world, it, rows, d, x, w, dev):
    s = torch.zeros(rows, d, dtype=torch.float32, device=dev)
    for r in range(world):
        s = s + _partial(r, it, rows, d, dev).float()
    x_new = x + s.half()
    f = x_new.float()
    h = (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + 1e-5)).half() * w
    return x_new, h


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from qfactory.comm import PeerComm
        from qfactory.decoder import DecoderConfig, QuantDecoder, teacher_forced_logits

        rows, d = 3, 2048
        comm = PeerComm.from_process_group(d, 16, dev)
        w = (torch.rand(d, generator=torch.Generator(device=dev).manual_seed(5), device=dev) + 0.5).half()
        x = torch.zeros(rows, d, dtype=torch.float16, device=dev)
        x_ref = x.clone()
        ok = True
        for it in range(40):                                  # launched one by one, slots alternating
            slot = it & 1
            comm.slot(slot, rows).copy_(_partial(rank, it, rows, d, dev))
            h = comm.allreduce_add_rmsnorm(slot, x, w, rows)
            x_ref, h_ref = _expected(world, it, rows, d, x_ref, w, dev)
            ok &= bool(torch.equal(x, x_ref)) and bool((h.float() - h_ref.float()).abs().max() <= 2e-3 * h_ref.float().abs().max())
        # the same from a CUDA graph of four reductions, replayed with new partials every time
        parts = [torch.zeros(rows, d, dtype=torch.float16, device=dev) for _ in range(4)]
        outs = [torch.empty(rows, d, dtype=torch.float16, device=dev) for _ in range(4)]
        st = torch.cuda.Stream(device=dev)
        st.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(st):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for j in range(4):
                    comm.slot(j & 1, rows).copy_(parts[j])
                    comm.allreduce_add_rmsnorm(j & 1, x, w, rows, out=outs[j])
        torch.cuda.current_stream(dev).wait_stream(st)
        for rep in range(5):
            for j in range(4):
                parts[j].copy_(_partial(rank, 100 + 4 * rep + j, rows, d, dev))
            g.replay()
            torch.cuda.synchronize(dev)
            for j in range(4):
                x_ref, h_ref = _expected(world, 100 + 4 * rep + j, rows, d, x_ref, w, dev)
                ok &= bool((outs[j].float() - h_ref.float()).abs().max() <= 2e-3 * h_ref.float().abs().max())
            ok &= bool(torch.equal(x, x_ref))
        status = comm.read_status()
        comm.close()
        # the sharded decoder against the unsharded one (same seeded network, same tokens)
        cfg = DecoderConfig(layers=2, d_model=1024, n_heads=8, n_kv_heads=8, d_ff=4096, vocab=2048, max_len=128, scale_boost=40.0)
        toks = torch.randint(0, cfg.vocab, (2, 84), generator=torch.Generator(device=dev).manual_seed(7), device=dev)
        tp = QuantDecoder(cfg, world=world, rank=rank, device=dev, seed=11, batch=2, weights="seeded")
        got = teacher_forced_logits(tp, toks, prompt_len=80).float()
        fused = tp.comm is not None
        # the same steps with the reductions received inside the consuming GEMVs (step-numbered exchange)
        tp.fuse_collect = True
        got_c = teacher_forced_logits(tp, toks, prompt_len=80).float()
        status_c = tp.comm.read_status() if tp.comm is not None else -1
        tp.close()
        one = QuantDecoder(cfg, world=1, rank=0, device=dev, seed=11, batch=2, weights="seeded")
        want = teacher_forced_logits(one, toks, prompt_len=80).float()
        rel = float((got - want).abs().max() / want.abs().max())
        rel_c = float((got_c - want).abs().max() / want.abs().max())
        ret[rank] = (ok, status, rel, fused, rel_c, status_c)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_memory_allreduce_and_tensor_parallel_decoder_between_real_ranks():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    for r in range(world):
        ok, status, rel, fused, rel_c, status_c = ret[r]
        assert ok and status == 0
        assert fused, "the peer buffers could not be mapped: the decoder fell back to NCCL"
        assert rel <= 2e-2
        assert rel_c <= 2e-2 and status_c == 0
