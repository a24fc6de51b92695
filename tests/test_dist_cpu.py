"""Multi-process logic on CPU ranks (gloo, world size 2): process groups and collectives, expert parallelism over the
all-to-all path against a single-rank run, a dynamic placement round with a real expert swap between ranks, and
host-side failure detection (a peer that never joins a collective ends it with an error, not a hang)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn(fn, world, *args):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, q, args)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    for _ in range(world):
        r, val = q.get(timeout=180)
        out[r] = val
    for p in procs:
        p.join(timeout=60)
    for r, v in out.items():
        if isinstance(v, str) and v.startswith("ERROR"):
            raise AssertionError(f"rank {r}: {v}")
    return out


_ONE_RANK: dict = {}


def _single(fn, *args):
    """Result of a one-rank run, computed once per (function, arguments): several cases compare against the same one."""
    key = (fn.__name__, repr(args))
    if key not in _ONE_RANK:
        _ONE_RANK[key] = _spawn(fn, 1, *args)[0]
    return _ONE_RANK[key]


def _entry(fn, rank, world, port, q, args):
    sys.path.insert(0, ROOT)
    torch.set_num_threads(1)        # several ranks share the cores; the models are tiny
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NO_GPU_MOCK="1")
    try:
        q.put((rank, fn(rank, world, *args)))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, "ERROR " + traceback.format_exc()[-1500:]))


# ---------------------------------------------------------------------------------------------- collectives
def _collectives(rank, world):
    from omni_infer_b200.parallel import destroy_distributed, init_distributed
    ps = init_distributed(backend="gloo", tp_size=2, dense_mlp_tp_size=2)
    g = ps.group("tp")
    x = torch.full((4, 3), float(rank + 1))
    assert torch.equal(g.all_reduce(x.clone()), torch.full((4, 3), 3.0))
    ag = g.all_gather(x)
    assert ag.shape == (8, 3) and ag[0, 0] == 1 and ag[4, 0] == 2
    rs = g.reduce_scatter(torch.arange(8.).view(4, 2))
    assert torch.equal(rs, (2 * torch.arange(8.).view(4, 2))[rank * 2:(rank + 1) * 2])
    a2a = g.all_to_all(torch.arange(4.) + 10 * rank)
    assert a2a.tolist() == ([0, 1, 10, 11] if rank == 0 else [2, 3, 12, 13])
    sw = g.swap(torch.tensor([float(rank)]))
    assert sw.item() == 1 - rank
    assert ps.dp_size == 1 and ps.tp_rank == rank and ps.ep_size == 2
    destroy_distributed()
    return "ok"


def test_groups_and_collectives():
    assert set(_spawn(_collectives, 2).values()) == {"ok"}


# ---------------------------------------------------------------------------------------------- two-level collectives
def _hierarchical(rank, world, rpd):
    from omni_infer_b200.parallel import destroy_distributed, init_distributed
    from omni_infer_b200.parallel import hierarchical as hc
    ps = init_distributed(backend="gloo", ranks_per_domain=rpd)
    hg, flat = ps.hier, ps.group("world")
    assert hg is not None and hg.ranks_per_domain == rpd and hg.num_domains == world // rpd
    assert hg.local.ranks == list(range(rank // rpd * rpd, rank // rpd * rpd + rpd))
    assert hg.cross.ranks == list(range(rank % rpd, world, rpd))
    assert hg.domain == rank // rpd and hg.local_index == rank % rpd
    g = torch.Generator().manual_seed(5 + rank)
    x = torch.randn(3, 10, generator=g)
    for dim in (0, 1):
        assert torch.equal(hc.all_gather_two_stage(x, hg, dim), flat.all_gather(x, dim))
    for chunks in (1, 2, 3):
        assert torch.equal(hc.all_gather_pipelined(x, hg, chunks), flat.all_gather(x, 0))
    y = torch.randint(-8, 8, (world * 2, 5, 4), generator=g).float()        # integers: sums are exact in any order
    want = flat.reduce_scatter(y)
    assert torch.equal(hc.reduce_scatter_two_stage(y, hg), want)
    for chunks in (2, 7):
        assert torch.equal(hc.reduce_scatter_pipelined(y, hg, chunks), want)
    z = torch.randint(-8, 8, (world * 3 + 1,), generator=g).float()         # element count not divisible by L
    for t in (y, z):
        assert torch.equal(hc.all_reduce_two_stage(t.clone(), hg), flat.all_reduce(t.clone()))
    if (world // rpd) & (world // rpd - 1) == 0:           # power-of-two domains: the pairwise rounds
        assert torch.equal(hc.all_gather_round_pipelined(x, hg), flat.all_gather(x, 0))
    else:
        with pytest.raises(ValueError):
            hc.all_gather_round_pipelined(x, hg)
    a = torch.arange(world * 2 * 3, dtype=torch.float32).view(world * 2, 3) + 1000 * rank
    assert torch.equal(hc.all_to_all_two_stage(a, hg), flat.all_to_all(a))
    # the process-wide forms pick the two-stage route by themselves
    assert torch.equal(hc.world_all_gather(x), flat.all_gather(x))
    assert torch.equal(hc.world_all_gather(x, pipelined_chunks=2), flat.all_gather(x))
    assert torch.equal(hc.world_reduce_scatter(y), want)
    assert torch.equal(hc.world_all_reduce(z.clone()), flat.all_reduce(z.clone()))
    assert torch.equal(hc.world_all_to_all(a), flat.all_to_all(a))
    assert hc.all_gather_local(x).shape[0] == 3 * rpd and hc.all_gather_cross(x).shape[0] == 3 * (world // rpd)
    assert hc.reduce_scatter_cross(hc.reduce_scatter_local(
        y.view(world // rpd, rpd, 2, 5, 4).transpose(0, 1).reshape(world * 2, 5, 4))).equal(want)
    assert hc.all_to_all_local(torch.arange(rpd * 2.)).shape[0] == rpd * 2
    destroy_distributed()
    return "ok"


@pytest.mark.parametrize("world,rpd", [(4, 2), (6, 3), (6, 2), (8, 2)])
def test_two_level_collectives_equal_the_flat_ones(world, rpd):
    assert set(_spawn(_hierarchical, world, rpd).values()) == {"ok"}


def test_one_domain_keeps_the_flat_route():
    from omni_infer_b200.parallel import hierarchical as hc
    from omni_infer_b200.parallel.parallel_state import get_parallel_state
    assert get_parallel_state().hier is None
    x = torch.arange(6.).view(3, 2)
    for f in (hc.world_all_gather, hc.world_reduce_scatter, hc.world_all_reduce, hc.world_all_to_all, hc.all_gather_cross,
              hc.reduce_scatter_cross):
        assert torch.equal(f(x), x)
    with pytest.raises(ValueError):
        hc.build_hierarchical_groups(8, 0, 3)


# ---------------------------------------------------------------------------------------------- linear family
def _linear_family(rank, world):
    """Every parallel linear against the dense product with the whole weight: shards cut by the layers' own slice
    functions, inputs sharded by token rows where the layer expects that."""
    from omni_infer_b200.layers import linear as L
    from omni_infer_b200.parallel import destroy_distributed, init_distributed
    ps = init_distributed(backend="gloo")
    g = ps.group("world")
    gen = torch.Generator().manual_seed(5)                       # same numbers on every rank
    T, H, N = 4 * world, 32, 24 * world
    x = torch.randn(T, H, generator=gen)
    rows = slice(rank * T // world, (rank + 1) * T // world)

    def fill(layer, full_w, full_b=None):
        with torch.no_grad():
            layer.weight.copy_(layer.weight.tp_slice_fn(full_w) if world > 1 else full_w)
            if full_b is not None:
                layer.bias.copy_(layer.bias.tp_slice_fn(full_b) if world > 1 else full_b)

    kw = dict(dtype=torch.float32)
    close = lambda a, b: torch.allclose(a, b, atol=1e-4, rtol=1e-4)      # noqa: E731
    # column parallel, rows gathered on the way in
    w, b = torch.randn(N, H, generator=gen), torch.randn(N, generator=gen)
    col = L.ColumnParallelFlashCommLinear(H, N, g, bias=True, **kw)
    fill(col, w, b)
    cols = slice(rank * N // world, (rank + 1) * N // world)
    assert close(col(x[rows].contiguous()), (x @ w.t() + b)[:, cols])
    # merged gate / up
    w2 = torch.randn(2 * N, H, generator=gen)
    mer = L.MergedColumnParallelFlashCommLinear(H, [N, N], g, **kw)
    fill(mer, w2)
    full = x @ w2.t()
    assert close(mer(x[rows].contiguous()), torch.cat([full[:, :N][:, cols], full[:, N:][:, cols]], 1))
    # row parallel: scatter back to row shards, or keep whole
    w3 = torch.randn(H, N, generator=gen)
    xin = torch.randn(T, N, generator=gen)
    for cls, red in ((L.RowParallelFlashCommLinear, "reduce_scatter"), (L.RowParallelLinearWithReduceScatter, "reduce_scatter"),
                     (L.RowParallelFlashCommLinear, "all_reduce"), (L.RowParallelLinearCross, "all_reduce")):
        row = cls(N, H, g, reduce=red, **kw) if cls is not L.RowParallelLinearWithReduceScatter else cls(N, H, g, **kw)
        fill(row, w3)
        want = xin @ w3.t()
        got = row(xin[:, cols].contiguous())
        assert close(got, want[rows] if row.reduce == "reduce_scatter" else want), cls.__name__
    assert L.RowParallelLinearCross(N, H, None, **kw).group is g                 # one domain: the world group
    # q / k / v with 4 query and 2 K/V heads (divided on 2 ranks, shared pairwise on 4)
    D, hq, hkv = 8, 4, 2
    wq = torch.randn((hq + 2 * hkv) * D, H, generator=gen)
    qkv = L.QKVParallelFlashCommLinear(H, D, hq, hkv, g, **kw)
    fill(qkv, wq)
    q, k, v = qkv(x[rows].contiguous())
    full = x @ wq.t()
    hql, hkvl, kv0 = hq // world, max(1, hkv // world), rank * hkv // world
    assert close(q, full[:, rank * hql * D:(rank + 1) * hql * D])
    assert close(k, full[:, hq * D + kv0 * D: hq * D + (kv0 + hkvl) * D])
    assert close(v, full[:, (hq + hkv) * D + kv0 * D:(hq + hkv) * D + (kv0 + hkvl) * D])
    # a whole block in the sequence-sharded form: gather -> column -> row -> scatter equals the dense block on my rows
    blk_in = L.ColumnParallelFlashCommLinear(H, N, g, **kw)
    blk_out = L.RowParallelFlashCommLinear(N, H, g, **kw)
    fill(blk_in, w)
    fill(blk_out, w3)
    assert close(blk_out(torch.relu(blk_in(x[rows].contiguous()))), (torch.relu(x @ w.t()) @ w3.t())[rows])
    destroy_distributed()
    return "ok"


@pytest.mark.parametrize("world", [2, 4])
def test_parallel_linear_family_equals_the_dense_product(world):
    assert set(_spawn(_linear_family, world).values()) == {"ok"}


# ---------------------------------------------------------------------------------------------- EP over all-to-all
def _ep_engine(rank, world, shared_ranks=0, overrides=None):
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams
    eng = EngineCore(EngineConfig(block_size=16, num_kv_blocks=32, max_model_len=128, device="cpu", seed=3,
                                  shared_expert_ranks=shared_ranks, model_overrides=dict(overrides or {})))
    if shared_ranks and world > 1:
        moe = eng.worker.runner.model.model.layers[1].mlp
        assert moe.shared_experts is None and moe.shared_ranks == shared_ranks
        assert moe.slots_per_rank == 8 // (world - shared_ranks)
        holds = [moe.logical_of_slot(s) for s in range(moe.slots_per_rank)]
        if rank < shared_ranks:      # shared pieces first, nothing else; no routed expert lives here
            assert holds[:moe.shared_pieces] == [("shared", j) for j in range(moe.shared_pieces)]
            assert all(h is None for h in holds[moe.shared_pieces:]) and not any(moe.local_slots_of(e) for e in range(8))
            assert float(moe.w13[moe.shared_pieces:].abs().sum()) == 0.0
        else:
            assert holds == list(range((rank - shared_ranks) * moe.slots_per_rank, (rank - shared_ranks + 1) * moe.slots_per_rank))
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 1024, (20,), generator=g).tolist() for _ in range(3)]
    ids = [eng.add_request(p, SamplingParams(max_tokens=6)) for p in prompts]
    outs = eng.run_until_done()
    if dist.is_initialized():
        dist.barrier()
    return [outs[i] for i in ids]


def test_expert_parallel_matches_single_rank():
    single = _single(_ep_engine)
    two = _spawn(_ep_engine, 2)
    assert two[0] == single and two[1] == single


@pytest.mark.parametrize("world,shared_ranks,overrides", [(2, 1, {}), (3, 1, {}), (4, 2, {}),
                                                          (3, 1, {"n_shared_experts": 2})])
def test_dedicated_shared_expert_ranks_match_single_rank(world, shared_ranks, overrides):
    """The first ranks hold only the shared expert (cut into pieces of a routed expert's shape, each an always-selected
    extra expert), the others only routed experts: same tokens as the model that runs everything on one rank."""
    single = _single(_ep_engine, 0, overrides)
    many = _spawn(_ep_engine, world, shared_ranks, overrides)
    assert all(many[r] == single for r in range(world))


def _ep_uneven(rank, world, mode, vocab_parallel=False):
    """Data-parallel ranks with different work: rank 0 serves three long requests, rank 1 one short request
    (mode "uneven") or none at all (mode "idle").  With multi-step decode and an MTP drafter the ranks need
    different numbers of model rounds per step; the agreement pads the quieter rank with dummy rounds."""
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams
    kw = dict(block_size=16, num_kv_blocks=48, max_model_len=160, device="cpu", seed=3, vocab_parallel=vocab_parallel)
    if mode == "async":
        kw.update(async_schedule=True, num_step=2)
    elif mode != "plain":
        kw.update(num_step=2, num_speculative_tokens=1, model_overrides={"num_nextn_predict_layers": 1})
    eng = EngineCore(EngineConfig(**kw))
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 1024, (20 + 3 * i,), generator=g).tolist() for i in range(3)]
    if world == 1 or rank == 0:
        ids = [eng.add_request(p, SamplingParams(max_tokens=9)) for p in prompts]
    elif mode == "idle":
        ids = []
    else:
        ids = [eng.add_request(prompts[1], SamplingParams(max_tokens=3))]
    outs = eng.run_until_done(max_steps=200)
    if dist.is_initialized():
        dist.barrier()
    return [outs[i] for i in ids]


def test_uneven_ranks_with_asynchronous_scheduling():
    """Asynchronous scheduling on two data-parallel ranks with different work: the rank that runs dry keeps executing
    dummy rounds on its worker thread, so the busy rank's exchanges always find their peer, and both leave together."""
    single = _single(_ep_uneven, "async")
    two = _spawn(_ep_uneven, 2, "async")
    assert two[0] == single and two[1] == [single[1][:3]]


@pytest.mark.parametrize("mode", ["uneven", "idle"])
def test_uneven_data_parallel_ranks_stay_in_step(mode):
    """Neither rank waits for an exchange its peer never joins, and the busy rank's tokens equal a single-rank run."""
    single = _single(_ep_uneven, mode)
    two = _spawn(_ep_uneven, 2, mode)
    assert two[0] == single
    if mode == "uneven":
        assert two[1] == [single[1][:3]]
    else:
        assert two[1] == []


def _vp_engine(rank, world, attn_tp, overrides=None):
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams
    eng = EngineCore(EngineConfig(block_size=16, num_kv_blocks=32, max_model_len=128, device="cpu", seed=3, attn_tp=attn_tp,
                                  tp_backend="nccl", vocab_parallel=True, model_overrides=dict(overrides or {})))
    if world > 1:
        m = eng.worker.runner.model
        per = (1024 + world - 1) // world
        assert m.model.embed_tokens.weight.shape[0] == per and m.lm_head.weight.shape[0] == per
        if rank == world - 1 and per * world > 1024:     # the rows past the vocabulary are zero
            assert float(m.lm_head.weight[1024 - per * (world - 1):].abs().sum()) == 0.0
    g = torch.Generator().manual_seed(11)
    n = 3 if (attn_tp or rank == 0) else 2               # data-parallel ranks with different numbers of requests
    prompts = [torch.randint(0, 1024, (17 + i,), generator=g).tolist() for i in range(3)][:n]
    ids = [eng.add_request(p, SamplingParams(max_tokens=6)) for p in prompts]
    outs = eng.run_until_done()
    if dist.is_initialized():
        dist.barrier()
    return [outs[i] for i in ids]


@pytest.mark.parametrize("world,attn_tp,overrides", [(2, False, {}), (3, False, {"n_routed_experts": 12}), (2, True, {})])
def test_vocabulary_parallel_table_and_head_match_single_rank(world, attn_tp, overrides):
    """Embedding table and LM head sharded by vocabulary rows (1024 rows over 3 ranks leaves a short last block): same
    tokens as one rank, with data-parallel attention (ranks hold different rows) and with tensor-parallel attention."""
    single = _single(_vp_engine, attn_tp, overrides)
    many = _spawn(_vp_engine, world, attn_tp, overrides)
    assert many[0] == single
    assert all(many[r] == single[:len(many[r])] for r in range(1, world))


def test_vocabulary_parallel_with_uneven_ranks_and_mtp():
    """Multi-step decode with a drafter on ranks with different work: the row-count agreement of the sharded table and
    head keeps the ranks in step, tokens equal the single-rank run."""
    single = _single(_ep_uneven, "uneven")
    two = _spawn(_ep_uneven, 2, "uneven", True)
    assert two[0] == single and two[1] == [single[1][:3]]


def _subgroup_engine(rank, world, mlp_tp, o_tp):
    """Data-parallel attention with the dense MLP / shared expert sharded over ``mlp_tp`` ranks and o_proj over
    ``o_tp`` ranks (all-gather -> MLP -> reduce-scatter; all-to-all -> o_proj -> reduce-scatter), uneven batches."""
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams
    eng = EngineCore(EngineConfig(block_size=16, num_kv_blocks=48, max_model_len=160, device="cpu", seed=3,
                                  dense_mlp_tp_size=mlp_tp, o_proj_tp_size=o_tp))
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 1024, (20 + 3 * i,), generator=g).tolist() for i in range(3)]
    mine = prompts if (world == 1 or rank == 0) else prompts[1:2]
    ids = [eng.add_request(p, SamplingParams(max_tokens=6)) for p in mine]
    outs = eng.run_until_done(max_steps=200)
    if dist.is_initialized():
        dist.barrier()
    return [outs[i] for i in ids]


@pytest.mark.parametrize("mlp_tp,o_tp", [(2, 1), (1, 2), (2, 2)])
def test_dense_mlp_and_o_proj_subgroups_match_single_rank(mlp_tp, o_tp):
    single = _single(_subgroup_engine, 1, 1)
    two = _spawn(_subgroup_engine, 2, mlp_tp, o_tp)
    assert two[0] == single and two[1] == [single[1]]


def _pp_engine(rank, world, model):
    """Two pipeline stages: each builds half of the layers, hidden states travel by point-to-point sends, the last
    stage samples and broadcasts the tokens; both stages are given the same requests."""
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams
    eng = EngineCore(EngineConfig(model=model, block_size=16, num_kv_blocks=48, max_model_len=160, device="cpu", seed=3,
                                  pp_size=world))
    if world > 1:
        m = eng.worker.runner.model.model
        assert (m.layer_lo, m.layer_hi) == ((0, 1) if rank == 0 else (1, 2)) or m.layer_hi - m.layer_lo >= 1
        assert eng.worker.runner.model.num_kv_layers == m.layer_hi - m.layer_lo
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 1024, (18 + 5 * i,), generator=g).tolist() for i in range(3)]
    ids = [eng.add_request(p, SamplingParams(max_tokens=6)) for p in prompts]
    outs = eng.run_until_done(max_steps=200)
    if dist.is_initialized():
        dist.barrier()
    return [outs[i] for i in ids]


@pytest.mark.parametrize("model", ["tiny-deepseek-v3", "tiny-qwen3-moe"])
def test_pipeline_parallel_matches_single_rank(model):
    single = _single(_pp_engine, model)
    two = _spawn(_pp_engine, 2, model)
    assert two[0] == single and two[1] == single


def test_pipeline_layer_ranges():
    from omni_infer_b200.parallel.pipeline import layer_range
    for n, pp in ((61, 4), (27, 2), (48, 8), (2, 2), (5, 3)):
        spans = [layer_range(n, r, pp) for r in range(pp)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1
    assert [layer_range(61, r, 4) for r in range(4)] == [(0, 15), (15, 31), (31, 46), (46, 61)]


# ---------------------------------------------------------------------------------------------- TP attention
def _tp_engine(rank, world, model="tiny-deepseek-v3", overrides=None):
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams
    eng = EngineCore(EngineConfig(model=model, model_overrides=dict(overrides or {}), block_size=16, num_kv_blocks=32,
                                  max_model_len=128, device="cpu", seed=3, attn_tp=True, tp_backend="nccl"))
    if world > 1 and not eng.model_cfg.use_mla:        # every rank caches its own K/V heads only
        from omni_infer_b200.layers.gqa import shard_heads
        want = shard_heads(eng.model_cfg.num_attention_heads, eng.model_cfg.num_key_value_heads, world, rank)[1]
        assert eng.worker.runner.kv_caches[0][0].shape[2] == want
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 1024, (17 + i,), generator=g).tolist() for i in range(3)]   # 56 rows: not a multiple of 8
    ids = [eng.add_request(p, SamplingParams(max_tokens=6)) for p in prompts]
    outs = eng.run_until_done()
    if dist.is_initialized():
        dist.barrier()
    return [outs[i] for i in ids]


def test_tensor_parallel_attention_matches_single_rank():
    """Heads sharded over two ranks, hidden states sharded by token rows between layers (library collectives on CPU):
    same tokens as the unsharded model."""
    single = _single(_tp_engine)
    two = _spawn(_tp_engine, 2)
    assert two[0] == single and two[1] == single


@pytest.mark.parametrize("world,overrides", [(2, {}), (2, {"num_key_value_heads": 1}), (4, {})])
def test_tensor_parallel_gqa_attention_matches_single_rank(world, overrides):
    """The GQA MoE model with query and K/V heads sharded over the ranks: K/V heads divided (4 q / 2 kv heads on 2 ranks),
    one K/V head shared by both ranks, and 2 K/V heads replicated over 4 ranks; same tokens as the unsharded model."""
    single = _single(_tp_engine, "tiny-qwen3-moe", overrides)
    many = _spawn(_tp_engine, world, "tiny-qwen3-moe", overrides)
    assert all(many[r] == single for r in range(world))


# ---------------------------------------------------------------------------------------------- everything at once
def _mixed_features_engine(rank, world, case):
    """Ranks with different requests and a KV pool that forces preemption, with the engine options of ``case`` on."""
    import random
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams
    case = dict(case)
    mtp, attn_tp = case.pop("mtp", False), case.pop("attn_tp", False)
    over = {"num_nextn_predict_layers": 1} if mtp else {}
    if world == 1:                                    # the baseline: plain options, roomy pool, one request at a time
        kw = dict(num_kv_blocks=64)
    else:
        kw = dict(case, attn_tp=attn_tp, tp_backend="nccl", **({"num_speculative_tokens": 1} if mtp else {}))
    eng = EngineCore(EngineConfig(block_size=16, max_model_len=128, device="cpu", seed=3, max_num_seqs=4, model_overrides=over, **kw))

    def jobs_of(r):
        r = 0 if attn_tp else r                       # tensor-parallel attention: every rank serves the same requests
        g, jr = torch.Generator().manual_seed(77 + r), random.Random(5 + r)
        shared = torch.randint(0, 1024, (32,), generator=g).tolist()
        return [((shared[: jr.choice([0, 16, 32])] + torch.randint(0, 1024, (jr.randint(1, 40),), generator=g).tolist())[:60],
                 jr.randint(1, 12)) for _ in range(jr.randint(1, 5))]

    if world == 1:
        table = {}
        for r in range(4):
            table[r] = []
            for p, n in jobs_of(r):
                i = eng.add_request(p, SamplingParams(max_tokens=n))
                table[r].append(eng.run_until_done()[i])
        return table
    jobs = jobs_of(rank)
    ids = [eng.add_request(p, SamplingParams(max_tokens=n)) for p, n in jobs]
    outs = eng.run_until_done(max_steps=5000)
    leak = eng.kv.num_free_blocks != kw["num_kv_blocks"] - 1
    if dist.is_initialized():
        dist.barrier()
    return {"outs": [outs[i] for i in ids], "leak": leak, "preemptions": eng.scheduler.stats["preemptions"]}


@pytest.mark.parametrize("world,case", [
    (2, dict(num_kv_blocks=9, enable_prefix_caching=True, enable_chunked_prefill=True, max_num_batched_tokens=24, num_step=3,
             async_schedule=True)),
    (4, dict(num_kv_blocks=10, num_step=3, mtp=True, attn_tp=True, vocab_parallel=True)),
    (2, dict(num_kv_blocks=9, enable_chunked_prefill=True, max_num_batched_tokens=24, num_step=2, mtp=True, vocab_parallel=True)),
], ids=["dp2-async-chunked-prefix-multistep", "tp4-mtp-multistep-vocab-parallel", "dp2-mtp-chunked-vocab-parallel"])
def test_engine_options_together_on_several_ranks(world, case):
    """The engine options that each have their own test, together, on ranks with different work and KV pools small
    enough to preempt: every request gets the tokens it gets when served alone by a plain one-rank engine."""
    base_key = {k: case[k] for k in ("mtp", "attn_tp") if k in case}
    want = _single(_mixed_features_engine, base_key)
    got = _spawn(_mixed_features_engine, world, case)
    for r in range(world):
        assert got[r]["outs"] == (want[0] if case.get("attn_tp") else want[r]), r
        assert not got[r]["leak"]
    assert sum(got[r]["preemptions"] for r in range(world)) > 0


# ---------------------------------------------------------------------------------------------- placement across ranks
def _placement_round(rank, world, host_replica=""):
    from omni_infer_b200.accelerators.placement import OmniPlanner
    from omni_infer_b200.layers.moe import MoELayer
    from omni_infer_b200.models.config import tiny_deepseek_v3
    from omni_infer_b200.parallel import destroy_distributed, init_distributed
    init_distributed(backend="gloo")
    cfg = tiny_deepseek_v3()
    pl = OmniPlanner(num_moe_layers=1, num_experts=8, max_redundant_per_rank=1, enable_dynamic=False, host_replica=host_replica,
                     _new=True)
    layer = MoELayer(cfg, 1, dtype=torch.float32, planner=pl)
    model = torch.nn.ModuleList([layer])
    with torch.no_grad():
        for s in range(layer.slots_per_rank):           # slot contents identify the expert they hold
            e = pl.logical_of_slot(0, s)
            layer.w13[s].fill_(float(e))
            layer.w2[s].fill_(float(e))
    pl.init_dram_weights(model)
    # expert 0 (on rank 0) is very hot
    pl.sent_counts[0, 0] = 5000 if rank == 0 else 4000
    pl.sent_counts[0, 1] = 10
    pl.sent_counts[0, 5] = 10
    if host_replica:
        import torch.distributed as dist
        dist.barrier()                                   # every rank of the host has filled its part of the replica
    n = pl.run_round()
    applied = pl.apply_pending()
    ins = pl.last_instructions()
    sel = pl.selector(0).tolist()
    spare = float(layer.w13[4, 0, 0])                    # the redundant slot of this rank
    place = pl.mapping.placement()[0].tolist()
    OmniPlanner.cleanup()
    destroy_distributed()
    return {"n": n, "applied": applied, "ins": ins, "sel": sel, "spare": spare, "place": place}


def _placement_round_replica(rank, world):
    return _placement_round(rank, world, host_replica=f"/omni_pytest_replica_{os.getppid()}")


def _background_placement_engine(rank, world, dynamic):
    """Decode while the planner's own thread runs placement rounds every 50 ms and the runner applies them between
    steps: skewed routing makes the balancer move experts all the time."""
    import time as _t
    from omni_infer_b200.accelerators.placement import OmniPlanner
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams
    pc = {"max_redundant_per_rank": 2, "enable_dynamic": True, "period_s": 0.05, "apply_interval": 1} if dynamic else None
    eng = EngineCore(EngineConfig(block_size=16, num_kv_blocks=64, max_model_len=160, device="cpu", seed=3,
                                  placement_config=pc, model_overrides={"router_skew": {"s": 1.2, "strength": 6.0, "seed": 0}}))
    g = torch.Generator().manual_seed(11 + rank)            # different requests on every rank
    prompts = [torch.randint(0, 1024, (20 + i,), generator=g).tolist() for i in range(3)]
    ids = [eng.add_request(p, SamplingParams(max_tokens=80, ignore_eos=True)) for p in prompts]
    outs = {}
    for _ in range(400):
        if not eng.has_unfinished and not eng.peers_busy:
            break
        for r in eng.step():
            outs.setdefault(r.request_id, []).extend(r.new_token_ids)
        if dynamic:
            _t.sleep(0.02)                                   # give the background rounds time to happen during the run
    planner = eng.worker.runner.planner
    applied = planner.applied_total if planner is not None else 0
    rounds = planner.ready_rounds() if planner is not None else 0
    if dist.is_initialized():
        dist.barrier()
    if planner is not None:
        OmniPlanner.cleanup()
    return {"outs": [outs[i] for i in ids], "applied": applied, "rounds": rounds}


def test_background_placement_rounds_never_change_the_tokens():
    """Experts are copied and re-routed between steps while requests decode.  A rank that re-routed to a replica before
    its holder had the weights would compute with an empty expert: every token must equal the run without placement."""
    plain = _spawn(_background_placement_engine, 2, False)
    moved = _spawn(_background_placement_engine, 2, True)
    assert moved[0]["applied"] + moved[1]["applied"] > 0 and moved[0]["rounds"] >= 2
    for r in range(2):
        assert moved[r]["outs"] == plain[r]["outs"], r


def test_dynamic_placement_round_moves_a_hot_expert():
    out = _spawn(_placement_round, 2)
    r0, r1 = out[0], out[1]
    assert r0["place"] == r1["place"]                    # both ranks agree on the new placement
    assert r0["n"] >= 1 and any(i["type"] == 1 and i["source_expert"] == 0 for i in r0["ins"])   # ADD of expert 0
    assert r1["place"][9] == 0                           # replica landed in rank 1's redundant slot (position 5+4)
    assert r1["spare"] == 0.0 and r1["applied"] >= 1     # with expert 0's weights
    assert r1["sel"][0] == 9 and r0["sel"][0] == 0       # every rank routes expert 0 to its own replica


def test_placement_round_from_the_host_replica():
    """Same round with the experts replicated once per host in shared memory: the rank that wants the hot expert copies
    it from there; the result is the same placement, weights and selectors as with the transfer between ranks."""
    out = _spawn(_placement_round_replica, 2)
    r0, r1 = out[0], out[1]
    assert r0["place"] == r1["place"] and r1["place"][9] == 0
    assert r1["spare"] == 0.0 and r1["applied"] >= 1
    assert r1["sel"][0] == 9 and r0["sel"][0] == 0


# ---------------------------------------------------------------------------------------------- failure detection
def _absent_peer(rank, world):
    import datetime
    if rank == 1:
        return "absent"                                   # this rank never joins
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        dist.barrier()
        return "no error"
    except Exception as e:  # noqa: BLE001
        return "detected: " + type(e).__name__


def _peer_stops_stepping(rank, world):
    import time as _t
    os.environ["OMNI_AGREE_TIMEOUT_S"] = "1.5"
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams
    eng = EngineCore(EngineConfig(block_size=16, num_kv_blocks=32, max_model_len=128, device="cpu", seed=3))
    eng.add_request(list(range(1, 20)), SamplingParams(max_tokens=200 if rank == 0 else 3, ignore_eos=True))
    if rank == 1:
        for _ in range(6):
            eng.step()                      # a few steps with its peer, then this rank stops stepping (a stuck host thread)
        _t.sleep(6.0)
        return "stopped"
    t0, steps = _t.time(), 0
    try:
        while eng.has_unfinished and _t.time() - t0 < 30:
            eng.step()
            steps += 1
        return f"no error after {steps} steps"
    except RuntimeError as e:
        return f"detected after {_t.time() - t0:.1f}s and {steps} steps: {str(e)[:60]}"


def test_a_peer_that_stops_stepping_ends_the_step_with_an_error():
    """Host-side failure detection in serving: the per-step agreement waits a bounded time for the peers (1.5 s here),
    then the step fails with a message that says so - the API server turns that into errors for its clients and, when
    it persists, into an unhealthy instance - instead of waiting out the process group's ten minutes."""
    out = _spawn(_peer_stops_stepping, 2)
    assert out[1] == "stopped"
    assert out[0].startswith("detected") and "did not join the step agreement" in out[0], out[0]
    waited = float(out[0].split()[2].rstrip("s"))
    assert waited < 6.0


def test_missing_rank_is_reported_not_hung():
    out = _spawn(_absent_peer, 2)
    assert out[1] == "absent" and out[0].startswith("detected")
