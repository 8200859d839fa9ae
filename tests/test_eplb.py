"""Expert-parallel load balancing on CPU: the placement policy evens out a skewed load, logical → physical mapping spreads a hot
expert over its replicas, and two gloo ranks shuffle expert weights to a new placement."""
import torch
import torch.multiprocessing as mp


def test_rebalance_evens_out_a_skewed_load():
    from onecat_vllm.parallel.eplb import EplbConfig, EplbState, map_to_physical, rebalance_experts
    g = torch.Generator().manual_seed(0)
    L, E, R = 3, 16, 4
    load = (torch.rand(L, E, generator=g) * 10).long() + 1
    load[:, 3] = 400                                           # one very hot expert per layer
    st = EplbState(L, E, R, EplbConfig(num_redundant_experts=4))
    before = st.balancedness(load)
    st.phy2log, st.log2phy, st.logcnt = rebalance_experts(load, st.P, R)
    after = st.balancedness(load)
    assert after > before and after > 0.55, (before, after)
    assert int(st.logcnt[0, 3]) >= 4                            # the redundant slots went to the hot expert
    for l in range(L):                                          # every logical expert has at least one slot; maps are consistent
        assert sorted(set(st.phy2log[l].tolist())) == list(range(E))
        for e in range(E):
            for p in st.log2phy[l, e][st.log2phy[l, e] >= 0].tolist():
                assert int(st.phy2log[l, p]) == e
    ids = torch.full((64, 2), 3)
    phys = map_to_physical(ids, st.log2phy[0], st.logcnt[0])
    assert set(phys.unique().tolist()) == set(st.log2phy[0, 3][st.log2phy[0, 3] >= 0].tolist())   # all replicas are used
    assert (st.phy2log[0][phys] == 3).all()
    st.record(0, torch.randint(0, E, (10, 2), generator=g))
    assert int(st.load()[0].sum()) == 20 and not st.step()


def _shuffle_rank(rank, port, q):
    import torch.distributed as dist
    from onecat_vllm.parallel.eplb import rearrange_expert_weights, rebalance_experts
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=2)
    L, E, P, R = 2, 6, 8, 2
    per = P // R
    old, _, _ = rebalance_experts(torch.ones(L, E), P, R)
    load = torch.tensor([[50, 1, 1, 1, 30, 1], [1, 1, 60, 1, 1, 1]])
    new, _, _ = rebalance_experts(load, P, R)
    # expert e of layer l carries the value 100 l + e in both of its weight tensors
    w = [[torch.stack([torch.full((3, 2), 100.0 * l + int(old[l, rank * per + i])) for i in range(per)]),
          torch.stack([torch.full((4,), 100.0 * l + int(old[l, rank * per + i])) for i in range(per)])] for l in range(L)]
    rearrange_expert_weights(old, new, w, rank, R)
    ok = all(bool((w[l][0][i] == 100.0 * l + int(new[l, rank * per + i])).all() and (w[l][1][i] == 100.0 * l + int(new[l, rank * per + i])).all())
             for l in range(L) for i in range(per))
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, ok, not torch.equal(old, new)))


def test_expert_weights_follow_the_new_placement_across_two_ranks():
    from onecat_vllm.executor.multiproc import _free_port
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_shuffle_rank, args=(r, port, q)) for r in range(2)]
    [p.start() for p in ps]
    [p.join(120) for p in ps]
    res = [q.get(timeout=5) for _ in range(2)]
    assert all(ok for _, ok, _ in res) and all(changed for _, _, changed in res), res
