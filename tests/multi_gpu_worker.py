"""Worker body of the multi-GPU tests: run under torchrun, one rank per GPU.
Compares the native device collectives and the fused kernels against NCCL
(`torch.distributed`) on the same inputs."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def check_collectives():
    from distdl_b200.parallel import collectives as C
    world, rank = dist.get_world_size(), dist.get_rank()
    ranks = list(range(world))
    dev = torch.device("cuda", torch.cuda.current_device())
    for dtype in (torch.bfloat16, torch.float32):
        for n in (8, 1000, 1001, 4096, 65536 + 24, 3 * 1024 * 1024 + 8):
            torch.manual_seed(n + rank)
            x = (torch.rand(n, device=dev) * 2 - 1).to(dtype)
            ref = x.clone().float()
            dist.all_reduce(ref)
            got = C.all_reduce(x, ranks)
            tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
            assert (got.float() - ref).abs().max().item() < tol * world, ("all_reduce", dtype, n)
            g = C.all_gather(x, ranks)
            refg = torch.empty(world, n, dtype=dtype, device=dev)
            dist.all_gather_into_tensor(refg, x)
            assert torch.equal(g, refg), ("all_gather", dtype, n)
            xs = (torch.rand(world, n, device=dev) * 2 - 1).to(dtype)
            rs = C.reduce_scatter(xs, ranks)
            refrs = torch.empty(n, dtype=torch.float32, device=dev)
            dist.reduce_scatter_tensor(refrs, xs.float().contiguous())
            assert (rs.float() - refrs).abs().max().item() < tol * world, ("reduce_scatter", dtype, n)
            a2a = C.all_to_all(xs, ranks)
            refa = torch.empty_like(xs)
            dist.all_to_all_single(refa, xs.contiguous())
            assert torch.equal(a2a, refa), ("all_to_all", dtype, n)
    # a sub-team (first two ranks) while the others idle
    if world >= 4:
        sub = [0, 1]
        if rank in sub:
            x = torch.full((1024,), float(rank + 1), device=dev)
            got = C.all_reduce(x, sub)
            assert torch.allclose(got, torch.full_like(got, 3.0))
    torch.cuda.synchronize()
    from distdl_b200 import _native
    assert _native.read_status()[0] == 0


def check_primitives_native():
    """The primitive modules on the native backend against their definition."""
    import distdl_b200
    from distdl_b200.nn import AllGather, AllSumReduce, ReduceScatter, Repartition
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    P_world = distdl_b200.backends.backend.Partition()
    P = P_world.create_cartesian_topology_partition([1, world])
    x = torch.full((4, 6), float(rank + 1), device=dev, dtype=torch.float32, requires_grad=True)
    y = AllSumReduce(P, axes_reduce=(1,))(x)
    assert torch.allclose(y, torch.full_like(y, world * (world + 1) / 2))
    y.sum().backward()
    assert torch.allclose(x.grad, torch.full_like(x.grad, float(world)))
    g = AllGather(P, axes_all_gather=(1,))(x.detach())
    assert g.shape == (4, 6 * world) and torch.allclose(g[:, 6 * rank:6 * rank + 6], x.detach())
    r = ReduceScatter(P, axes_reduce_scatter=(1,))(torch.ones(4, 2 * world, device=dev))
    assert r.shape == (4, 2) and torch.allclose(r, torch.full_like(r, float(world)))
    # row partition -> column partition transpose of an [N, N] tensor
    N = 8 * world
    P_rows = P_world.create_cartesian_topology_partition([world, 1])
    G = torch.arange(N * N, device=dev, dtype=torch.float32).reshape(N, N)
    rows = G[rank * 8:(rank + 1) * 8].clone()
    cols = Repartition(P_rows, P)(rows)
    assert torch.equal(cols, G[:, rank * 8:(rank + 1) * 8])
    # halo exchange along a 1-D chain of all GPUs: ghosts receive the neighbours' values
    from distdl_b200.nn import HaloExchange
    P_chain = P_world.create_cartesian_topology_partition([1, 1, world])
    hl, hr = int(rank > 0), int(rank < world - 1)
    halo = [[0, 0], [0, 0], [hl, hr]]
    t = torch.zeros(2, 3, 5 + hl + hr, device=dev)
    t[:, :, hl:hl + 5] = float(rank + 1)
    t.requires_grad_()
    out = HaloExchange(P_chain, halo, halo, halo)(t)
    if hl:
        assert torch.all(out[:, :, 0] == float(rank))
    if hr:
        assert torch.all(out[:, :, -1] == float(rank + 2))
    out.sum().backward()
    want = torch.ones_like(t)
    if hl:
        want[:, :, 0] = 0
        want[:, :, hl] = 2
    if hr:
        want[:, :, -1] = 0
        want[:, :, -1 - hr] = 2
    assert torch.equal(t.grad, want)


def check_box_exchange():
    """The one-kernel halo exchange and repartition against the same primitives on the library path
    (NCCL point-to-point + PyTorch slicing): messages of several chunks, faces with and without a
    contiguous run, corners over two phases, the adjoint's add-and-clear in bf16, many calls in a row
    (buffers and counters are reused)."""
    import numpy as np

    import distdl_b200
    from distdl_b200.backends.common.functional import halo_exchange as hx
    from distdl_b200.backends.common.transport import GroupTransport
    from distdl_b200.nn import HaloExchange, Repartition
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    be = distdl_b200.backends.backend
    native, plain = be.transport(), GroupTransport()
    assert getattr(native, "box_plan", None) is not None
    P_world = be.Partition()
    # ---- halo exchange on a [1, 1, a, b] grid (a * b = world), widths 1 and 2
    a = 2 if world % 2 == 0 else 1
    grid = [1, 1, a, world // a]
    P = P_world.create_cartesian_topology_partition(grid)
    halo = np.array([[0, 0], [0, 0], [1, 1], [2, 2]])
    idx = P.index
    for d in (2, 3):
        if idx[d] == 0:
            halo[d][0] = 0
        if idx[d] == grid[d] - 1:
            halo[d][1] = 0
    layer = HaloExchange(P, halo, halo, halo)
    for dtype, bulk in ((torch.float32, (64, 52)), (torch.bfloat16, (33, 40)), (torch.float32, (256, 260))):
        shape = [4, 16] + [bulk[d - 2] + int(halo[d][0]) + int(halo[d][1]) for d in (2, 3)]
        torch.manual_seed(7 + rank)
        x = torch.randn(*shape, device=dev).to(dtype)
        layer._distdl_module_setup((x,))
        for rep in range(3):
            for fn in (hx.fill_ghosts, hx.fold_ghosts):
                want = fn(plain, x, P, layer.slices, layer.neighbor_ranks)
                got = fn(native, x, P, layer.slices, layer.neighbor_ranks)
                if dtype == torch.float32:
                    assert torch.equal(want, got), ("halo", fn.__name__, dtype, bulk, rep)
                else:
                    assert torch.allclose(want.float(), got.float(), atol=3e-2, rtol=2e-2), ("halo", fn.__name__, rep)
            x = x + 1
    # ---- repartition: row blocks -> column blocks of an [N, N] tensor, small and multi-chunk
    P_rows = P_world.create_cartesian_topology_partition([world, 1])
    P_cols = P_world.create_cartesian_topology_partition([1, world])
    for N, dtype in ((8 * world, torch.float32), (40 * world + 3, torch.float32), (1024 * world, torch.bfloat16),
                     (2048 * world, torch.float32)):
        layer = Repartition(P_rows, P_cols, preserve_batch=False)
        from distdl_b200.utilities.slicing import compute_start_index, compute_subshape
        lo = int(compute_start_index([world, 1], [rank, 0], [N, N])[0])
        n = int(compute_subshape([world, 1], [rank, 0], [N, N])[0])
        gen = torch.Generator(device=dev).manual_seed(3)
        full = torch.randn(N, N, device=dev, generator=gen).to(dtype)
        x = full[lo:lo + n].clone()
        for rep in range(3):
            y = layer(x)
            clo = int(compute_start_index([1, world], [0, rank], [N, N])[1])
            cn = int(compute_subshape([1, world], [0, rank], [N, N])[1])
            assert torch.equal(y, full[:, clo:clo + cn]), ("repartition", N, dtype, rep)
    from distdl_b200 import _native
    assert _native.read_status()[0] == 0


def check_multimem_allreduce():
    """The job-wide all-reduce through the NVLink multicast region (multimem.ld_reduce / multimem.st)
    against NCCL.  All comparisons are collected first and the region is torn down on every rank
    before anything is asserted, so that no rank leaves while its memory is still bound."""
    from distdl_b200 import _native
    from distdl_b200.parallel import collectives, symm
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    symm.heap()
    region = symm.enable_multicast(32 << 20)
    if region is None:
        if rank == 0:
            print("multicast objects are not supported here: skipped")
        return
    problems = []
    try:
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
            for n in (1024, 16 * 1024 + 8, 300_000, 3_000_000, 9_000_001):
                torch.manual_seed(100 + rank)
                x = (torch.rand(n, device=dev) * 2 - 1).to(dtype)
                want = x.float().clone()
                dist.all_reduce(want)
                for rep in range(2):
                    got = collectives.all_reduce(x, list(range(world))).float()
                    err = (got - want).abs().max().item() / (want.abs().max().item() + 1e-6)
                    if not err < tol:
                        problems.append((str(dtype), n, rep, err))
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
            for n in (512, 40_000, 2_000_003):
                torch.manual_seed(200 + rank)
                x = (torch.rand(world, n, device=dev) * 2 - 1).to(dtype)
                want = x.float().clone()
                dist.all_reduce(want)
                got = collectives.reduce_scatter(x, list(range(world))).float()
                err = (got - want[rank]).abs().max().item() / (want.abs().max().item() + 1e-6)
                if not err < tol:
                    problems.append(("reduce_scatter", str(dtype), n, err))
        status = _native.read_status()
        if status[0]:
            problems.append(("device status", status))
    except Exception as e:      # noqa: BLE001  (reported after the tear-down)
        problems.append(("exception", repr(e)))
    flags = [None] * world
    dist.all_gather_object(flags, problems)
    symm.disable_multicast()
    assert not any(flags), flags


def check_zero_grad_accumulate():
    """ZeRO weight gradients on the fast paths must equal the plain path (bf16 reduce-scatter
    by autograd): (1) unsharded fp32 accumulators filled by the weight-gradient GEMMs and
    reduce-scattered once, in place; (2) the reduce-scatter fused with scale + fp32
    accumulation after every micro-batch."""
    import os
    import distdl_b200
    from distdl_b200.nn import DistributedLinearAllGatherZero
    from distdl_b200.parallel import FlatAdamW
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([world, 1, 1])
    for full in ("1", "0"):
        os.environ["DISTDL_FULL_GRADS"] = full
        torch.manual_seed(5)
        a = DistributedLinearAllGatherZero(P, 256, 512, bias=False, dtype=torch.bfloat16)
        b = DistributedLinearAllGatherZero(P, 256, 512, bias=False, dtype=torch.bfloat16)
        b.load_state_dict(a.state_dict())
        opt = FlatAdamW(a, max_grad_norm=None)
        assert bool(opt._full) == (full == "1")
        torch.manual_seed(100 + rank)
        for _ in range(2):                                   # two micro-batches accumulate
            x = torch.randn(4, 64, 256, device=dev, dtype=torch.bfloat16)
            a(x).float().pow(2).sum().backward()
            b(x).float().pow(2).sum().backward()
        opt.reduce_gradients()
        assert a.weight.grad is None                          # never materialised as a bf16 gradient
        ref = b.weight.grad.float().reshape(-1)
        got = a.weight.main_grad_view
        err = (got - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
        assert err < 2e-2, (full, err)
    os.environ.pop("DISTDL_FULL_GRADS", None)


def check_split_norm():
    """Feature-split LayerNorm / RMSNorm with the fused statistics exchange against
    the serial fp32 norm of the concatenated features (unequal shards)."""
    from distdl_b200.parallel import split_norm
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    ranks = tuple(range(world))
    rows = 777
    d_r = 64 + 8 * (rank % 2)
    for rms in (False, True):
        torch.manual_seed(10 + rank)
        x = torch.randn(rows, d_r, device=dev).to(torch.bfloat16).requires_grad_()
        w = (1 + 0.1 * torch.randn(d_r, device=dev)).to(torch.bfloat16).requires_grad_()
        b = None if rms else (0.1 * torch.randn(d_r, device=dev)).to(torch.bfloat16).requires_grad_()
        dy = torch.randn(rows, d_r, device=dev).to(torch.bfloat16)
        parts = [None] * world
        dist.all_gather_object(parts, (x.detach().float().cpu(), w.detach().float().cpu(),
                                       None if b is None else b.detach().float().cpu(), dy.float().cpu()))
        n_global = sum(p[0].shape[1] for p in parts)
        assert split_norm.usable(x, w, b, ranks)
        y = split_norm.split_norm(x, w, b, 1e-5, ranks, n_global, rms=rms)
        y.backward(dy)
        xf = torch.cat([p[0] for p in parts], 1).requires_grad_()
        wf = torch.cat([p[1] for p in parts]).requires_grad_()
        bf = None if rms else torch.cat([p[2] for p in parts]).requires_grad_()
        dyf = torch.cat([p[3] for p in parts], 1)
        if rms:
            ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
        else:
            ref = torch.nn.functional.layer_norm(xf, (n_global,), wf, bf, 1e-5)
        ref.backward(dyf)
        lo = sum(p[0].shape[1] for p in parts[:rank])
        sl = slice(lo, lo + d_r)
        for got, want, what in ((y, ref[:, sl], "y"), (x.grad, xf.grad[:, sl], "dx"), (w.grad, wf.grad[sl], "dw")) + \
                (() if rms else ((b.grad, bf.grad[sl], "db"),)):
            want = want.detach().to(dev)
            err = (got.float() - want).abs().max().item() / (want.abs().max().item() + 1e-6)
            assert err < 2e-2, ("split_norm", rms, what, err)


def check_layernorm_module():
    """DistributedLayerNorm over a feature dimension split across all GPUs takes the fused
    kernel on the native backend and matches the serial LayerNorm (forward and input gradient)."""
    import distdl_b200
    from distdl_b200 import _native
    from distdl_b200.nn import DistributedLayerNorm
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    D = 64 * world
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([1, world])
    ln = DistributedLayerNorm(P, D, dtype=torch.bfloat16)
    torch.manual_seed(7)
    full = torch.randn(200, D, device=dev)
    dyf = torch.randn(200, D, device=dev)
    x = full[:, rank * 64:(rank + 1) * 64].to(torch.bfloat16).contiguous().requires_grad_()
    before = _native.launch_count
    y = ln(x)
    assert _native.launch_count > before, "the fused split-norm kernel did not run"
    y.backward(dyf[:, rank * 64:(rank + 1) * 64].to(torch.bfloat16))
    xf = full.to(torch.bfloat16).float().requires_grad_()
    ref = torch.nn.functional.layer_norm(xf, (D,), None, None, ln.eps)
    ref.backward(dyf.to(torch.bfloat16).float())
    sl = slice(rank * 64, (rank + 1) * 64)
    for got, want, what in ((y, ref[:, sl], "y"), (x.grad, xf.grad[:, sl], "dx")):
        err = (got.float() - want.detach()).abs().max().item() / (want.abs().max().item() + 1e-6)
        assert err < 2e-2, ("layernorm module", what, err)


def check_context_parallel_attention():
    """DistributedSelfAttention on GPUs: native point-to-point exchange for the head <-> sequence
    repartitions around the flash-attention kernels, against serial fp32 attention."""
    import distdl_b200
    from distdl_b200.nn import DistributedSelfAttention
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([1, world, 1, 1])
    att = DistributedSelfAttention(P, causal=True)
    b, s, hq, hkv, d = 2, 256 * world, 2 * world, world, 128
    torch.manual_seed(4)
    Q, K, V = (torch.randn(b, s, h, d, device=dev) for h in (hq, hkv, hkv))
    dO = torch.randn(b, s, hq, d, device=dev)
    sl = slice(rank * (s // world), (rank + 1) * (s // world))
    q, k, v = (t[:, sl].to(torch.bfloat16).contiguous().requires_grad_() for t in (Q, K, V))
    out = att(q, k, v)
    out.backward(dO[:, sl].to(torch.bfloat16).contiguous())
    Qr, Kr, Vr = (t.to(torch.bfloat16).float().requires_grad_() for t in (Q, K, V))
    rep = hq // hkv
    ref = torch.nn.functional.scaled_dot_product_attention(
        Qr.transpose(1, 2), Kr.transpose(1, 2).repeat_interleave(rep, 1), Vr.transpose(1, 2).repeat_interleave(rep, 1),
        is_causal=True).transpose(1, 2)
    ref.backward(dO.to(torch.bfloat16).float())
    for got, want, what in ((out, ref[:, sl], "out"), (q.grad, Qr.grad[:, sl], "dq"), (k.grad, Kr.grad[:, sl], "dk"),
                            (v.grad, Vr.grad[:, sl], "dv")):
        err = (got.float() - want.detach()).abs().max().item() / (want.abs().max().item() + 1e-6)
        assert err < 3e-2, ("context-parallel attention", what, err)


def check_ring_attention():
    """DistributedRingAttention on GPUs: the flash-attention kernels per (query block, key block)
    pair with the global log-sum-exp, ring hops over peer memory, against serial fp32 attention."""
    import distdl_b200
    from distdl_b200.nn import DistributedRingAttention
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([1, world, 1, 1])
    att = DistributedRingAttention(P, causal=True)
    b, s, hq, hkv, d = 2, 256 * world, 4, 2, 128
    torch.manual_seed(11)
    Q, K, V = (torch.randn(b, s, h, d, device=dev) for h in (hq, hkv, hkv))
    dO = torch.randn(b, s, hq, d, device=dev)
    sl = slice(rank * (s // world), (rank + 1) * (s // world))
    q, k, v = (t[:, sl].to(torch.bfloat16).contiguous().requires_grad_() for t in (Q, K, V))
    out = att(q, k, v)
    out.backward(dO[:, sl].to(torch.bfloat16).contiguous())
    Qr, Kr, Vr = (t.to(torch.bfloat16).float().requires_grad_() for t in (Q, K, V))
    rep = hq // hkv
    ref = torch.nn.functional.scaled_dot_product_attention(
        Qr.transpose(1, 2), Kr.transpose(1, 2).repeat_interleave(rep, 1), Vr.transpose(1, 2).repeat_interleave(rep, 1),
        is_causal=True).transpose(1, 2)
    ref.backward(dO.to(torch.bfloat16).float())
    for got, want, what in ((out, ref[:, sl], "out"), (q.grad, Qr.grad[:, sl], "dq"), (k.grad, Kr.grad[:, sl], "dk"),
                            (v.grad, Vr.grad[:, sl], "dv")):
        err = (got.float() - want.detach()).abs().max().item() / (want.abs().max().item() + 1e-6)
        assert err < 3e-2, ("ring attention", what, err)


def check_symmetric_params():
    """ZeRO shards gathered in place from the optimizer's peer-mapped buffer give the same
    training trajectory as the staged all-gather."""
    import os
    from distdl_b200 import models
    from distdl_b200.parallel import SyntheticTokens, Trainer
    world = dist.get_world_size()
    losses = {}
    for mode in ("0", "1"):
        os.environ["DISTDL_SYMM_PARAMS"] = mode
        torch.manual_seed(0)
        cfg = models.llama_tiny(d_model=256, n_heads=4, n_kv_heads=2, ffn_dim=512, max_seq=128, vocab_size=1024)
        layout = models.ParallelLayout(world, 1)
        model = models.Decoder(cfg, layout)
        trainer = Trainer(model, global_tokens_per_step=2 * world * 128, micro_batch=1, lr=2e-3, warmup_steps=0)
        assert trainer.opt._symmetric == (mode == "1"), "unexpected parameter placement"
        data = SyntheticTokens(2, 128, cfg.vocab_size, dp_index=layout.dp_index, seed=3)
        block = data.next()
        losses[mode] = [trainer.step(block).item() for _ in range(4)]
    os.environ.pop("DISTDL_SYMM_PARAMS", None)
    for a, b in zip(losses["0"], losses["1"]):
        assert abs(a - b) < 1e-3 * max(1.0, abs(a)), losses
    assert losses["1"][-1] < losses["1"][0], losses


def check_overlapped_gradient_step():
    """ZeRO gradients reduced block by block while the backward pass of the last micro-batch is still
    running (and, without clipping, applied by the fused reduce + AdamW kernel) against the same
    training with everything reduced inside the optimizer step."""
    import os
    from distdl_b200 import _native, models
    from distdl_b200.parallel import SyntheticTokens, Trainer
    world = dist.get_world_size()
    for clip in (1.0, 0.0):
        losses = {}
        for mode in ("0", "1"):
            os.environ["DISTDL_OVERLAP_GRADS"] = mode
            torch.manual_seed(0)
            cfg = models.llama_tiny(d_model=256, n_heads=4, n_kv_heads=2, ffn_dim=512, max_seq=128, vocab_size=1024)
            cfg.n_layers = 3
            layout = models.ParallelLayout(world, 1)
            model = models.Decoder(cfg, layout)
            trainer = Trainer(model, global_tokens_per_step=4 * world * 128, micro_batch=2, lr=2e-3, warmup_steps=0,
                              max_grad_norm=clip)
            assert bool(trainer.opt._by_block) == (mode == "1"), "unexpected grouping of the accumulators"
            data = SyntheticTokens(4, 128, cfg.vocab_size, dp_index=layout.dp_index, seed=3)
            block = data.next()
            launches = _native.launch_count
            losses[mode] = [trainer.step(block).item() for _ in range(4)]
            if mode == "1":
                assert len(trainer.opt._block_done) == 3      # every block was reduced from its backward hook
        os.environ.pop("DISTDL_OVERLAP_GRADS", None)
        for a, b in zip(losses["0"], losses["1"]):
            assert abs(a - b) < 1e-3 * max(1.0, abs(a)), (clip, losses)
        assert losses["1"][-1] < losses["1"][0], losses
    assert _native.read_status()[0] == 0


def check_moe_peer():
    """Expert-parallel block: dispatch / combine over peer memory against the unfused path
    (permutation kernels + all-to-all), outputs and all gradients."""
    import os
    from distdl_b200 import models
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    results = {}
    for mode in ("0", "1"):
        os.environ["DISTDL_MOE_PEER"] = mode
        torch.manual_seed(0)
        cfg = models.mixtral_tiny(n_experts=2 * world, d_model=256, ffn_dim=512, n_heads=4, n_kv_heads=2,
                                  vocab_size=512, max_seq=128, checkpoint_blocks=False, n_layers=1)
        lay = models.ParallelLayout(world, 1)
        m = models.Decoder(cfg, lay)
        moe = m.blocks[0].mlp
        torch.manual_seed(50 + rank)
        x = (torch.randn(2, 128, 256, device=dev) * 0.5).to(torch.bfloat16).requires_grad_()
        y = moe(x)
        (y.float() * torch.linspace(-1, 1, 256, device=dev)).sum().backward()
        results[mode] = (y.detach().float(), x.grad.float(), moe.w_up.grad.float(), moe.w_down.grad.float())
    os.environ.pop("DISTDL_MOE_PEER", None)
    for a, b, what in zip(results["0"], results["1"], ("y", "dx", "dw_up", "dw_down")):
        err = (a - b).abs().max().item() / (a.abs().max().item() + 1e-6)
        assert err < 2e-2, ("moe peer", what, err)


def check_context_parallel_decoder():
    """The decoder with a context-parallel size of 2 against the data-parallel decoder with the
    same shards fed whole sequences on both replicas (its loss and gradients are exactly twice
    those of the context-parallel model), in the three modes ring / zigzag ring / all-to-all.  bf16,
    head dim 128, blocks of 256 tokens (chunks of 128 in the zigzag layout): the rings run the tcgen05
    attention kernels per block and the rotary kernel with position offsets or ranges.
    Run by name only (``multi_gpu_worker.py context_decoder`` on an even number of GPUs)."""
    from distdl_b200 import models
    world = dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    tp = world // 2
    # the all-to-all mode re-splits the LOCAL heads over the context-parallel workers: 4 query and 2
    # key heads per tensor-parallel worker, head dim 128
    cfg = models.llama_tiny(d_model=512 * tp, n_heads=4 * tp, n_kv_heads=2 * tp, ffn_dim=1024 * tp, max_seq=512,
                            vocab_size=1024)
    cfg.n_layers = 2
    gen = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, cfg.vocab_size, (2, 513), generator=gen).to(dev)
    for mode in ("ring", "zigzag", "a2a"):
        cfg.cp_mode = mode
        torch.manual_seed(0)
        cp_model = models.Decoder(cfg, models.ParallelLayout(1, tp, cp=2))
        torch.manual_seed(0)
        dp_model = models.Decoder(cfg, models.ParallelLayout(2, tp))
        out = {}
        for name, model in (("cp", cp_model), ("dp", dp_model)):
            model.train()
            loss = model.loss(tokens[:, :-1], tokens[:, 1:], scale=1.0 / 1024)
            loss.backward()
            model.release_gathered()
            total = loss.detach().float().clone()
            dist.all_reduce(total)
            out[name] = (total, [None if p.grad is None else p.grad.float().clone() for p in model.parameters()])
        assert abs(float(out["cp"][0]) * 2 - float(out["dp"][0])) < 2e-2 * abs(float(out["dp"][0])), \
            (mode, float(out["cp"][0]), float(out["dp"][0]))
        for ga, gb in zip(out["cp"][1], out["dp"][1]):
            if ga is not None and ga.numel():
                err = (ga * 2 - gb).abs().max() / gb.abs().max().clamp_min(1e-6)
                assert err < 5e-2, (mode, float(err))


def check_activation_policies():
    """Tensor-parallel (x ZeRO on more than 2 GPUs) training with every block recomputing against every
    block keeping its activations (the fused kernels' gathered inputs stored, norm and activation
    outputs rebuilt, weights gathered again in backward): the same loss trajectory."""
    from distdl_b200 import models
    from distdl_b200.parallel import SyntheticTokens, Trainer
    world = dist.get_world_size()
    tp = 2 if world % 2 == 0 else 1
    losses = {}
    for policy in ("full", "none", "1"):
        torch.manual_seed(0)
        cfg = models.llama_tiny(d_model=512, n_heads=4, n_kv_heads=2, ffn_dim=1024, max_seq=256, vocab_size=1024)
        cfg.n_layers, cfg.activation_policy = 3, policy
        layout = models.ParallelLayout(world // tp, tp)
        model = models.Decoder(cfg, layout)
        trainer = Trainer(model, global_tokens_per_step=2 * (world // tp) * 256, micro_batch=1, lr=2e-3,
                          warmup_steps=0)
        data = SyntheticTokens(2, 256, cfg.vocab_size, dp_index=layout.dp_index, seed=3)
        block = data.next()
        losses[policy] = [trainer.step(block).item() for _ in range(4)]
        assert model.activation_plan["keep"] == {"full": 0, "none": 3, "1": 1}[policy]
    for policy in ("none", "1"):
        for a, b in zip(losses["full"], losses[policy]):
            assert abs(a - b) < 2e-3 * max(1.0, abs(a)), losses
    assert losses["none"][-1] < losses["none"][0], losses


def check_pipelined_decoder():
    """Two pipeline stages (of ``world / 2`` tensor-parallel workers each) train: the loss falls and
    no device wait runs out.  The schedule and the per-stage optimizer layout on GPUs."""
    from distdl_b200 import models
    from distdl_b200.parallel import SyntheticTokens, Trainer
    world = dist.get_world_size()
    if world % 2:
        return
    torch.manual_seed(0)
    cfg = models.llama_tiny(d_model=512, n_heads=4, n_kv_heads=2, ffn_dim=1024, max_seq=256, vocab_size=1024)
    cfg.n_layers = 4
    piped = models.PipelinedDecoder(cfg, pp=2, dp=1, tp=world // 2)
    trainer = Trainer(piped, global_tokens_per_step=4 * 256, micro_batch=1, lr=2e-3, warmup_steps=0)
    data = SyntheticTokens(4, 256, cfg.vocab_size, dp_index=0, seed=3)
    block = data.next()
    losses = [trainer.step(block).item() for _ in range(5)]
    assert losses[-1] < losses[0], losses
    from distdl_b200 import _native
    assert _native.read_status()[0] == 0


def main():
    import distdl_b200
    from distdl_b200.backends.common import world as dworld
    dworld.init_process_group_from_env()
    distdl_b200.config.set_backend("native", "cupy")
    what = sys.argv[1] if len(sys.argv) > 1 else "collectives"
    todo = set(what.split(","))                 # several groups in one launch: "all,activation_policies,multimem"
    run_all = "all" in todo
    if run_all or "collectives" in todo:
        check_collectives()
    if run_all or "primitives" in todo:
        check_primitives_native()
        check_zero_grad_accumulate()
        check_split_norm()
        check_layernorm_module()
        check_context_parallel_attention()
        check_ring_attention()
        check_symmetric_params()
        check_overlapped_gradient_step()
        check_moe_peer()
    if "context_decoder" in todo:
        check_context_parallel_decoder()
    if run_all or "box" in todo:
        check_box_exchange()
    if "activation_policies" in todo:
        check_activation_policies()
    if "pipeline" in todo:
        check_pipelined_decoder()
    if run_all or "fused" in todo:
        from multi_gpu_fused import check_fused
        check_fused()
    if "multimem" in todo:                      # last: binds the multicast region for the rest of the process
        check_multimem_allreduce()
    dist.barrier()
    if dist.get_rank() == 0:
        print(f"multi-gpu {what}: OK on {dist.get_world_size()} GPUs")
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback
        traceback.print_exc()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1)      # skip communicator destructors: a failed rank must not linger
