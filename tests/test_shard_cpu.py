"""The N>1 host logic on CPU: two gloo ranks.  N-column shards all-gathered
equal the unsharded product bit for bit; the expert-parallel all-to-all
dispatch/combine equals the single-rank block bit for bit (the reference
tests partitioned graphs the same way, against the unpartitioned result:
tests/unit/planner_partition_test.cc).  The per-rank arithmetic is the CPU
oracle here; on GPUs the same functions carry llmp_b200's kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, fn, out_dir):
    import sys
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        result = fn(rank, world)
        np.save(os.path.join(out_dir, f"r{rank}.npy"), result)
    finally:
        dist.destroy_process_group()


def _run(fn, tmp_path, world=2):
    mp.spawn(_worker, args=(world, _free_port(), fn, str(tmp_path)), nprocs=world, join=True)
    return [np.load(os.path.join(tmp_path, f"r{r}.npy")) for r in range(world)]


def _column_shards(rank, world):
    from llmp_b200 import shard, synth
    from oracle import binding as orc
    rng = np.random.default_rng(0)
    n, k, tokens = 40, 512, 3
    w = synth.q4_k_weights(rng, n, k)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    y = orc.quantize_q8_1(x)
    b, e = shard.row_shard(n, world, rank)
    mine = orc.vecq(orc.Q4_K, w[b:e], y, k, e - b, tokens, threads=1)[:, 0, :]
    sizes = [shard.row_shard(n, world, r)[1] - shard.row_shard(n, world, r)[0] for r in range(world)]
    return shard.all_gather_rows(torch.from_numpy(mine), sizes).numpy()


def test_n_column_shards_gather_to_the_unsharded_product(tmp_path, orc):
    from llmp_b200 import shard, synth
    got = _run(_column_shards, tmp_path)
    rng = np.random.default_rng(0)
    w = synth.q4_k_weights(rng, 40, 512)
    x = rng.normal(0, 1, size=(3, 512)).astype(np.float32)
    want = orc.vecq(orc.Q4_K, w, orc.quantize_q8_1(x), 512, 40, 3, threads=1)[:, 0, :]
    for r in range(2):
        assert np.array_equal(got[r], want)
    assert shard.row_shard(12288, 8, 3, multiple=128) == (4608, 6144)
    assert shard.row_shard(10, 4, 0) == (0, 3) and shard.row_shard(10, 4, 3) == (8, 10)
    with pytest.raises(ValueError):
        shard.row_shard(100, 2, 0, multiple=128)


def _expert_weights():
    from llmp_b200 import synth
    rng = np.random.default_rng(1)
    experts, hidden, inter = 6, 256, 256
    gate_up = synth.q4_k_weights(rng, experts * 2 * inter, hidden).reshape(experts, 2 * inter, -1)
    down = synth.q4_k_weights(rng, experts * hidden, inter).reshape(experts, hidden, -1)
    return experts, hidden, inter, gate_up, down


def _expert_rows(orc, gate_up, down, hidden, inter, rows, expert_ids):
    """Rows through their experts, one row at a time (row-independent arithmetic)."""
    out = np.zeros((rows.shape[0], hidden), np.float32)
    for i in range(rows.shape[0]):
        e = int(expert_ids[i])
        aq = orc.quantize_mmq_q8_1(rows[i:i + 1])
        gu = orc.mmq_q4_k(gate_up[e], aq, hidden, 2 * inter, threads=1)
        h = np.array([[orc.glu(orc.GLU_SWIGLU, gu[0, j], gu[0, inter + j]) for j in range(inter)]],
                     np.float32)
        out[i] = orc.mmq_q4_k(down[e], orc.quantize_mmq_q8_1(h), inter, hidden, threads=1)[0]
    return out


def _tokens(rank):
    from llmp_b200 import synth
    rng = np.random.default_rng(10 + rank)
    tokens, used = 5 + rank, 2
    ids, w = synth.topk_route(rng, tokens, 6, used)
    if rank == 0:
        ids[1, 1] = 7                       # an id outside the experts
    x = rng.normal(0, 1, size=(tokens, 256)).astype(np.float32)
    return x, ids, w


def _expert_parallel(rank, world):
    from llmp_b200 import shard
    from oracle import binding as orc
    experts, hidden, inter, gate_up, down = _expert_weights()
    b, e = shard.expert_range(experts, world, rank)
    x, ids, w = _tokens(rank)

    def local(rows, local_ids):
        return torch.from_numpy(_expert_rows(orc, gate_up[b:e], down[b:e], hidden, inter,
                                             rows.numpy(), local_ids.numpy()))

    return shard.ep_moe_ffn(torch.from_numpy(x), torch.from_numpy(ids), torch.from_numpy(w),
                            experts, local).numpy()


def test_expert_parallel_all_to_all_equals_one_rank(tmp_path, orc):
    got = _run(_expert_parallel, tmp_path)
    experts, hidden, inter, gate_up, down = _expert_weights()
    for rank in range(2):
        x, ids, w = _tokens(rank)
        tokens, used = ids.shape
        flat = ids.reshape(-1)
        rows = _expert_rows(orc, gate_up, down, hidden, inter, x[np.arange(tokens * used) // used],
                            flat.clip(0, experts - 1))
        position = np.where((flat >= 0) & (flat < experts), np.arange(tokens * used), -1)
        want = orc.moe_combine(rows, position.astype(np.int32), w, tokens, used)
        assert np.array_equal(np.isnan(got[rank]), np.isnan(want))
        ok = ~np.isnan(want)
        assert np.array_equal(got[rank][ok], want[ok])


def _expert_parallel_padded(rank, world):
    from llmp_b200 import shard
    from oracle import binding as orc
    experts, hidden, inter, gate_up, down = _expert_weights()
    b, e = shard.expert_range(experts, world, rank)
    x, ids, w = _tokens(rank)
    tokens, used = ids.shape
    capacity = 8                               # small: rank 1's seven-token batch overflows no lane

    def pack(xt, idt):
        send, send_ids, home, dropped = shard.pack_reference(xt, idt, experts, world, capacity)
        assert dropped == 0
        return send, send_ids, home

    def local(rows, local_ids):
        lid = local_ids.numpy()
        out = np.full((rows.shape[0], hidden), np.nan, np.float32)     # unused lanes: never read back
        live = lid >= 0
        out[live] = _expert_rows(orc, gate_up[b:e], down[b:e], hidden, inter, rows.numpy()[live],
                                 lid[live])
        return torch.from_numpy(out)

    def combine(back, home, wt):
        return torch.from_numpy(orc.moe_combine(back.numpy(), home.numpy(), wt.numpy(), tokens, used))

    return shard.ep_moe_ffn_padded(torch.from_numpy(x), torch.from_numpy(ids), torch.from_numpy(w),
                                   experts, capacity, pack, local, combine).numpy()


def test_fixed_capacity_expert_parallel_equals_one_rank(tmp_path, orc):
    """The exchange of fixed-size lanes (the form the GPUs run: no split size ever reaches the
    host) gives the single-rank block bit for bit, ids outside the experts included."""
    from llmp_b200 import shard
    got = _run(_expert_parallel_padded, tmp_path)
    experts, hidden, inter, gate_up, down = _expert_weights()
    for rank in range(2):
        x, ids, w = _tokens(rank)
        tokens, used = ids.shape
        flat = ids.reshape(-1)
        rows = _expert_rows(orc, gate_up, down, hidden, inter, x[np.arange(tokens * used) // used],
                            flat.clip(0, experts - 1))
        position = np.where((flat >= 0) & (flat < experts), np.arange(tokens * used), -1)
        want = orc.moe_combine(rows, position.astype(np.int32), w, tokens, used)
        assert np.array_equal(np.isnan(got[rank]), np.isnan(want))
        ok = ~np.isnan(want)
        assert np.array_equal(got[rank][ok], want[ok])
    assert shard.ep_capacity(1024, 8, 8) == 1280 and shard.ep_capacity(1, 8, 8) == 128
    # a lane that overflows drops rows and says so
    x, ids, _ = _tokens(1)
    _, _, home, dropped = shard.pack_reference(torch.from_numpy(x), torch.from_numpy(ids), 6, 2, 2)
    assert dropped > 0 and int((home < 0).sum()) == dropped
