"""Behaviour that a program written against the reference relies on, checked on CPU ranks:
identity short-cuts, inactive workers, zero-volume outputs, where roots and parameters live, how
``scale_backward`` acts, lazy re-setup on a changed input, world-size independent embedding
initialisation, and the loss value living on worker 0."""
import torch

from dist_harness import run_ranks


def _P(ranks, shape):
    import distdl_b200 as d
    return d.backends.backend.Partition().create_partition_inclusive(ranks).create_cartesian_topology_partition(shape)


def body_identities_and_inactive(rank, world):
    from distdl_b200.nn import (AllGather, AllSumReduce, Broadcast, HaloExchange, ReduceScatter, Repartition,
                                SumReduce)
    from distdl_b200.utilities.torch import zero_volume_tensor
    x = torch.randn(3, 4, requires_grad=True)
    # one-worker partitions: the collective modules return their input object itself
    P1 = _P([rank], [1, 1])
    for layer in (AllGather(P1, axes_all_gather=(0,)), ReduceScatter(P1, axes_reduce_scatter=(0,)),
                  AllSumReduce(P1, axes_reduce=(0,)), HaloExchange(P1, [[0, 0], [0, 0]], [[0, 0], [0, 0]],
                                                                   [[0, 0], [0, 0]])):
        assert layer(x) is x, type(layer).__name__
    # equal partitions: broadcast / sum-reduce are identities (values equal; a copy is allowed)
    P = _P([0, 1, 2, 3], [2, 2])
    for cls in (Broadcast, SumReduce):
        y = cls(P, P)(x)
        assert torch.equal(y, x), cls.__name__
    assert torch.equal(Repartition(P, P)(x), x)
    # workers outside both partitions get their input back from the modules
    P_a, P_b = _P([0], [1, 1]), _P([0, 1], [1, 2])
    if rank >= 2:
        z = zero_volume_tensor()
        assert Broadcast(P_a, P_b)(z) is z and SumReduce(P_b, P_a)(z) is z
        assert AllGather(P_b, axes_all_gather=(1,))(z) is z
    # a worker that is active in the input but holds no output gets a zero-volume tensor, which
    # keeps the batch dimension with preserve_batch=True
    if rank < 2:
        xin = torch.randn(5, 2, requires_grad=True)
        y = SumReduce(P_b, P_a, preserve_batch=True)(xin)
        y2 = SumReduce(P_b, P_a, preserve_batch=False)(xin)
        if rank == 0:
            assert y.shape == (5, 2) and y2.shape == (5, 2)
        else:
            assert tuple(y.shape) == (5, 0) and y2.numel() == 0 and y2.dim() == 1
    return True


def test_identity_shortcuts_inactive_workers_and_zero_volume_outputs():
    run_ranks("test_behaviour", "body_identities_and_inactive", 4, timeout=180)


def body_roots_and_scale_backward(rank, world):
    from distdl_b200.nn import AllGather, AllSumReduce, Broadcast, DistributedLinearAllGather
    from distdl_b200.utilities.torch import zero_volume_tensor
    # the root of a broadcast is the FIRST worker of the source partition, whatever its world rank
    P_src, P_dst = _P([2], [1]), _P([2, 0, 1, 3], [4])
    x = torch.full((2,), 7.0, requires_grad=True) if rank == 2 else zero_volume_tensor(requires_grad=True)
    y = Broadcast(P_src, P_dst, preserve_batch=False)(x)
    assert torch.equal(y, torch.full((2,), 7.0))
    # scale_backward is a scalar divisor of the incoming gradient; None means gradients are SUMMED
    P = _P([0, 1, 2, 3], [4])
    for scale, want in ((None, 4.0), (4, 1.0), (2, 2.0)):
        x = torch.ones(3, requires_grad=True)
        AllSumReduce(P, axes_reduce=(0,), scale_backward=scale)(x).sum().backward()
        assert torch.allclose(x.grad, torch.full((3,), want)), (scale, x.grad)
    x = torch.ones(2, requires_grad=True)
    AllGather(P, axes_all_gather=(0,), scale_backward=4)(x).sum().backward()
    assert torch.allclose(x.grad, torch.ones(2))               # 4 copies summed, divided by 4
    # parameters live on the storing partition only; everybody else holds zero-volume BUFFERS of the
    # same names that require grad, so the key sets of state_dict() agree on all workers
    P_feat = _P([0, 1, 2, 3], [2, 1, 2])
    lin = DistributedLinearAllGather(P_feat, 6, 8)
    names = dict(lin.named_parameters())
    if int(P_feat.index[0]) == 0:
        assert tuple(lin.weight.shape) == (1, 4, 6) and "weight" in names and "bias" in names
    else:
        assert lin.weight.numel() == 0 and lin.weight.requires_grad and "weight" not in names
        assert "weight" in dict(lin.named_buffers())
    assert set(lin.state_dict()) == {"weight", "bias"}
    return True


def test_roots_scale_backward_and_parameter_placement():
    run_ranks("test_behaviour", "body_roots_and_scale_backward", 4, timeout=180)


def body_lazy_setup(rank, world):
    """The structure of the input is re-examined at every call: a changed shape rebuilds the layer's
    buffers and output shape; with the check switched off the first structure is kept."""
    import distdl_b200
    from distdl_b200.nn import AllGather
    P = _P([0, 1, 2, 3], [1, 4])
    layer = AllGather(P, axes_all_gather=(1,))
    assert tuple(layer(torch.ones(2, 3)).shape) == (2, 12)
    assert tuple(layer(torch.ones(5, 2)).shape) == (5, 8)          # new structure -> new setup
    calls = []
    orig = layer._distdl_module_setup
    layer._distdl_module_setup = lambda inp: (calls.append(1), orig(inp))[1]
    layer(torch.ones(5, 2))
    assert not calls                                                # same structure: no new setup
    layer(torch.ones(1, 2))
    assert calls == [1]
    old = distdl_b200.config.check_input_changed if hasattr(distdl_b200.config, "check_input_changed") else None
    return old is None or bool(old) in (True, False)


def test_setup_is_lazy_and_keyed_by_the_input_structure():
    run_ranks("test_behaviour", "body_lazy_setup", 4, timeout=180)


def body_embedding_init(rank, world, shape):
    from distdl_b200.nn import DistributedEmbedding, Repartition
    torch.manual_seed(11)                                           # every worker: same seed
    P = _P(list(range(world)), shape)
    emb = DistributedEmbedding(P, 10, 8, collect_state=True)
    sd = emb.state_dict()
    return sd["weight"].clone() if rank == 0 else None


def test_embedding_initialisation_does_not_depend_on_the_worker_grid():
    a = run_ranks("test_behaviour", "body_embedding_init", 4, args=([2, 1, 2],), timeout=180)[0]
    b = run_ranks("test_behaviour", "body_embedding_init", 4, args=([1, 1, 4],), timeout=180)[0]
    c = run_ranks("test_behaviour", "body_embedding_init", 2, args=([1, 1, 2],), timeout=180)[0]
    assert torch.equal(a, b) and torch.equal(a, c)


def body_loss_on_root(rank, world):
    from distdl_b200.nn import DistributedMSELoss
    P = _P([0, 1, 2, 3], [2, 2])
    torch.manual_seed(rank)
    x = torch.randn(3, 2, requires_grad=True)
    t = torch.zeros(3, 2)
    loss = DistributedMSELoss(P)(x, t)
    loss.backward()                                                 # every worker calls backward
    import torch.distributed as dist
    sq = (x.detach() ** 2).sum()
    dist.all_reduce(sq)
    assert loss.dim() == 0
    if rank == 0:
        assert torch.allclose(loss, sq / 24)                        # mean over the 4 x 6 global entries
    else:
        assert float(loss) == 0.0                                   # a stand-in scalar
    assert torch.allclose(x.grad, 2 * x.detach() / 24, atol=1e-6)   # but the gradient is the true one
    return True


def test_loss_value_lives_on_the_first_worker_gradients_everywhere():
    run_ranks("test_behaviour", "body_loss_on_root", 4, timeout=180)


def body_reset_setup(rank, world):
    """A shape change that only one worker can see: 4 + 3 entries, then 4 + 4.  Worker 0's input looks the
    same both times, so the layer's collective set-up has to be requested explicitly on all workers."""
    from distdl_b200.nn import AllGather, reset_setup
    P = _P([0, 1], [2])
    layer = AllGather(P, axes_all_gather=(0,))
    y = layer(torch.full((4 if rank == 0 else 3,), float(rank)))
    assert y.tolist() == [0.0] * 4 + [1.0] * 3
    reset_setup(layer)
    assert not layer._distdl_is_setup
    y = layer(torch.full((4,), float(rank)))
    assert y.tolist() == [0.0] * 4 + [1.0] * 4 and layer._distdl_is_setup
    return True


def test_reset_setup_for_changes_one_worker_cannot_see():
    run_ranks("test_behaviour", "body_reset_setup", 2, timeout=120)
