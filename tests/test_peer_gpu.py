"""The peer-store exchange (llmp_b200_peer_*): on one GPU, with the ranks emulated in one
process and every kernel run to completion before the next is queued, so that no kernel here
ever waits for another kernel of the same GPU; the wait's give-up path by a flag nobody sets."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _pair(world, vectors, sites):
    from llmp_b200 import peer
    ranks = [peer.PeerExchange(world, r, vectors, sites) for r in range(world)]
    everyone = [x.pointers() for x in ranks]
    for x in ranks:
        x.connect(everyone)
    return ranks


def test_slices_published_by_every_rank_are_what_the_gathered_quantizer_reads(cuda):
    torch = cuda
    import llmp_b200 as ops
    world, n = 2, 1536
    ranks = _pair(world, {"h": n}, sites=3)
    rng = np.random.default_rng(5)
    for step in range(3):                      # flags carry the step number: replays must work
        whole = torch.from_numpy(rng.normal(0, 1, size=n).astype(np.float32)).cuda()
        want = ops.quantize_q8(whole.view(1, n))
        for x in ranks:
            x.begin_step()
        torch.cuda.synchronize()
        per = n // world
        for r, x in enumerate(ranks):
            x.publish("h", 1, whole[r * per:(r + 1) * per].contiguous(), r * per)
        torch.cuda.synchronize()               # every flag is set before any wait is queued
        for x in ranks:
            got = torch.empty_like(want)
            x.quantize_q8("h", 1, got)
            torch.cuda.synchronize()
            assert torch.equal(got, want), step
            assert torch.equal(x.vectors["h"], whole)
            assert not x.timed_out()
            assert int(x.step.item()) == step + 1
    assert ops.device_faults() == 0
    for x in ranks:
        x.close()


def test_publish_wait_and_quantize_in_one_launch(cuda):
    torch = cuda
    import llmp_b200 as ops
    world, n = 2, 2560
    ranks = _pair(world, {"y": n}, sites=2)
    rng = np.random.default_rng(6)
    whole = torch.from_numpy(rng.normal(0, 1, size=n).astype(np.float32)).cuda()
    other = torch.from_numpy(rng.normal(0, 1, size=512).astype(np.float32)).cuda()
    per = n // world
    for x in ranks:
        x.begin_step()
    torch.cuda.synchronize()
    ranks[1].publish("y", 1, whole[per:].contiguous(), per)
    torch.cuda.synchronize()                   # rank 1's flag is set before rank 0 waits for it
    got = torch.empty((1, ops.q8_1_row_blocks(n) * 36), dtype=torch.uint8, device="cuda")
    ranks[0].exchange_quantize_q8("y", 1, whole[:per].contiguous(), 0, got)
    torch.cuda.synchronize()
    assert torch.equal(got, ops.quantize_q8(whole.view(1, n)))
    assert torch.equal(ranks[1].vectors["y"], whole)      # rank 0's slice reached rank 1 too
    # the exchange as back-pressure only: another input is quantized once the flags are there
    got2 = torch.empty((1, ops.q8_1_row_blocks(512) * 36), dtype=torch.uint8, device="cuda")
    ranks[1].quantize_q8("y", 1, got2, x=other)
    torch.cuda.synchronize()
    assert torch.equal(got2, ops.quantize_q8(other.view(1, 512)))
    assert not ranks[0].timed_out() and not ranks[1].timed_out() and ops.device_faults() == 0
    for x in ranks:
        x.close()


def _pair_words(world, words):
    from llmp_b200 import peer
    ranks = [peer.PeerExchange(world, r, {}, 1, words=words) for r in range(world)]
    everyone = [x.pointers() for x in ranks]
    for x in ranks:
        x.connect(everyone)
    return ranks


@pytest.mark.parametrize("n,k,glu", [(10240, 2560, True), (2560, 10240, False)])
def test_products_fan_their_rows_out_as_tagged_words(cuda, n, k, glu):
    """The two dense decode kernels store token 0's results, tagged, into every rank's vector;
    the word quantizer gives the Q8_1 blocks of exactly those values, for two steps running."""
    torch = cuda
    import llmp_b200 as ops
    from llmp_b200 import synth
    world = 2
    ranks = _pair_words(world, {"h": n})
    rng = np.random.default_rng(n)
    per = n // world
    w = torch.from_numpy(synth.q4_k_weights(rng, n, k)).cuda()
    g = torch.from_numpy(synth.q4_k_weights(rng, n, k)).cuda() if glu else None
    for step in range(2):
        x = torch.from_numpy(rng.normal(0, 1, size=(1, k)).astype(np.float32)).cuda()
        q8 = ops.quantize_q8(x)
        for r in ranks:
            r.begin_step()
        shards = []
        for r, ex in enumerate(ranks):
            rows = slice(r * per, (r + 1) * per)
            out = ops.vecq(w[rows].contiguous(), ops.TYPE_Q4_K, k, per, q8, 1,
                           gate=g[rows].contiguous() if glu else None,
                           glu=ops.GLU_GEGLU if glu else ops.GLU_NONE, fan=ex.fan("h", r * per, 7))
            shards.append(out)
        torch.cuda.synchronize()               # every word is there before any reader polls
        whole = torch.cat(shards, dim=1)
        want = ops.quantize_q8(whole)
        for ex in ranks:
            assert torch.equal(ex.word_values("h", 0, n), whole.view(-1)), step
            got = torch.empty_like(want)
            ex.quantize_words(got, name="h", first=0, count=n, tag=7)
            torch.cuda.synchronize()
            assert torch.equal(got, want), step
            # ... and as back-pressure only: x is quantized once the held words are there
            got_x = torch.empty_like(q8)
            ex.quantize_words(got_x, x=x, hold=("h", 0, n, 7))
            torch.cuda.synchronize()
            assert torch.equal(got_x, q8)
            assert not ex.timed_out()
    assert ops.device_faults() == 0
    # a tag nobody stored: the reader gives up and says so
    before = ops.device_faults()
    ranks[0].quantize_words(torch.empty_like(want), name="h", first=0, count=n, tag=9, polls=20)
    torch.cuda.synchronize()
    assert ranks[0].timed_out() and ops.device_faults() > before
    ops.device_faults_clear()
    for ex in ranks:
        ex.close()


def test_a_wait_for_a_flag_nobody_sets_gives_up_and_says_so(cuda):
    torch = cuda
    import llmp_b200 as ops
    ranks = _pair(2, {"y": 256}, sites=2)
    before = ops.device_faults()
    a = ranks[0]
    a.begin_step()
    a.publish("y", 0, torch.ones(128, device="cuda"), 0)     # rank 1 never publishes
    torch.cuda.synchronize()
    a.wait("y", 0, polls=50)
    torch.cuda.synchronize()
    assert a.timed_out()
    assert ops.device_faults() == before + 1
    out = torch.empty((1, ops.q8_1_row_blocks(256) * 36), dtype=torch.uint8, device="cuda")
    a.quantize_q8("y", 1, out, polls=20)                     # the fused form: same give-up path
    torch.cuda.synchronize()
    assert a.timed_out()
    assert ops.device_faults() == before + 2
    ops.device_faults_clear()
    # the context is intact: an ordinary launch afterwards is correct
    x = torch.randn((1, 512), device="cuda")
    assert ops.quantize_q8(x).shape[1] == ops.q8_1_row_blocks(512) * 36
    torch.cuda.synchronize()
    for r in ranks:
        r.close()


def test_publish_refuses_what_it_cannot_copy(cuda):
    torch = cuda
    import llmp_b200 as ops
    (x,) = _pair(1, {"h": 64}, sites=1)
    with pytest.raises(ops.Rejected):
        x.publish("h", 0, torch.ones(16, device="cuda"), 3)          # offset not 16-byte aligned
    with pytest.raises(ops.Rejected):
        x.publish("h", 1, torch.ones(16, device="cuda"), 0)          # no such site
    torch.cuda.synchronize()
    x.close()
