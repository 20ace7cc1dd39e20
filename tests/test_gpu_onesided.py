"""One-sided transfers and the device-initiated replica weight channel, with all logical ranks of
the group emulated on one GPU (kernels of different ranks are ordered by the stream, never by
waiting on one another).  Expected values come from plain PyTorch indexing."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worlds(n, arena=8 << 20):
    from ep_balance_b200.parallel.onesided import SymmetricWorld

    return SymmetricWorld.local(n, arena, torch.device("cuda", 0))


@pytest.mark.parametrize("use_bulk", [True, False])
def test_get_put_batched_match_indexing(use_bulk):
    worlds = _worlds(4)
    try:
        n = 3 * 8192 + 4096 + 48          # several tiles plus a ragged end, 16-byte multiple
        sym = [w.create_tensor((6, n), torch.uint8) for w in worlds]
        for r, t in enumerate(sym):
            t.copy_(torch.randint(0, 255, (6, n), dtype=torch.uint8, device="cuda"))
        ref = [t.clone() for t in sym]
        me = worlds[1]
        me.use_bulk = use_bulk
        local = torch.zeros((5, n), dtype=torch.uint8, device="cuda")
        off = me.offset_of(sym[1])
        desc = torch.tensor([[0, off + 2 * n, 0 * n, n], [3, off + 5 * n, 1 * n, n], [-1, 0, 2 * n, n],
                             [1, off + 0 * n, 3 * n, n], [2, off + 1 * n + 16, 4 * n + 32, n - 64]],
                            dtype=torch.int64, device="cuda")
        me.get_batched(local, desc, blocks=3)
        torch.cuda.synchronize()
        assert torch.equal(local[0], ref[0][2]) and torch.equal(local[1], ref[3][5])
        assert int(local[2].sum()) == 0
        assert torch.equal(local[3], ref[1][0])
        assert torch.equal(local[4][32:32 + n - 64], ref[2][1][16:16 + n - 64])
        assert int(local[4][:32].sum()) == 0 and int(local[4][n - 32:].sum()) == 0

        src = torch.randint(0, 255, (2, n), dtype=torch.uint8, device="cuda")
        pdesc = torch.tensor([[2, off + 4 * n, 0, n], [0, off + 3 * n, n, n]], dtype=torch.int64, device="cuda")
        me.put_batched(src, pdesc, blocks=2)
        torch.cuda.synchronize()
        assert torch.equal(sym[2][4], src[0]) and torch.equal(sym[0][3], src[1])
        assert torch.equal(sym[2][3], ref[2][3])     # neighbours untouched
        me.check_status()
    finally:
        worlds[0].destroy()


def test_unaligned_ranges_take_the_byte_path():
    worlds = _worlds(2, arena=1 << 20)
    try:
        sym = [w.create_tensor((4096,), torch.uint8) for w in worlds]
        sym[1].copy_(torch.arange(4096, device="cuda").to(torch.uint8))
        local = torch.zeros(4096, dtype=torch.uint8, device="cuda")
        w0 = worlds[0]
        off = w0.offset_of(sym[0])
        desc = torch.tensor([[1, off + 3, 5, 1001]], dtype=torch.int64, device="cuda")
        w0.get_batched(local, desc)
        torch.cuda.synchronize()
        assert torch.equal(local[5:5 + 1001], sym[1][3:3 + 1001])
        assert int(local[:5].sum()) == 0 and int(local[5 + 1001:].sum()) == 0
    finally:
        worlds[0].destroy()


def test_get_put_single_and_signals():
    worlds = _worlds(3, arena=1 << 20)
    try:
        sym = [w.create_tensor((256, 64), torch.bfloat16) for w in worlds]
        for r, t in enumerate(sym):
            t.fill_(float(r + 1))
        assert worlds[0].is_symmetric_tensor(sym[0]) and not worlds[0].is_symmetric_tensor(torch.zeros(4, device="cuda"))
        dst = torch.zeros((256, 64), dtype=torch.bfloat16, device="cuda")
        worlds[0].get(dst, sym[0], peer=2)
        torch.cuda.synchronize()
        assert float(dst.float().mean()) == 3.0
        worlds[0].put_signal(sym[0], torch.full((256, 64), 9.0, dtype=torch.bfloat16, device="cuda"), peer=1, idx=5)
        worlds[2].signal(1, 5, 2)
        worlds[1].wait_signal(5, 3)        # already satisfied: returns at once
        torch.cuda.synchronize()
        assert float(sym[1].float().mean()) == 9.0
        assert worlds[1].test_signal(5) == 3 and worlds[0].test_signal(5) == 0
        worlds[1].check_status()
        worlds[0].signal(-1, 7)
        torch.cuda.synchronize()
        assert [w.test_signal(7) for w in worlds] == [1, 1, 1]
    finally:
        worlds[0].destroy()


def test_wait_on_a_signal_nobody_sends_reports_status():
    worlds = _worlds(2, arena=1 << 16)
    try:
        worlds[0].wait_signal(9, 1)        # emulation: zero budget, the wait gives up immediately
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="code=2"):
            worlds[0].check_status()
        worlds[0].check_status()           # status was cleared; the context is still usable
        assert int(torch.ones(4, device="cuda").sum()) == 4
    finally:
        worlds[0].destroy()


def test_replica_weight_channel_matches_indexing():
    from ep_balance_b200.parallel.symm_weights import SymmReplicaTransport, SymmWeightReplicator

    R, E, n_slot = 4, 8, 4
    shapes = [(16, 32), (32, 8)]
    dtype = torch.bfloat16
    main = torch.arange(E) // (E // R)
    x = torch.zeros((E, R), dtype=torch.int8)
    x[torch.arange(E), main] = 1
    x[0, 2] = 1
    x[0, 3] = 1
    x[5, 0] = 1
    arena = SymmWeightReplicator.arena_bytes(E, R, shapes, dtype, n_slot=n_slot)
    worlds = _worlds(R, arena=arena)
    try:
        g = torch.Generator(device="cuda").manual_seed(0)
        params = {e: tuple(torch.randn(s, generator=g, device="cuda").to(dtype) for s in shapes) for e in range(E)}
        reps = [SymmWeightReplicator(w, main, shapes, dtype) for w in worlds]
        trs = [SymmReplicaTransport(reps[r], x.cuda(), n_slot,
                                    {e: params[e] for e in range(E) if int(main[e]) == r}) for r in range(R)]
        # forward, phase by phase over the logical ranks
        for t in trs:
            t.publish()
        stacks = [t.pull() for t in trs]
        torch.cuda.synchronize()
        for r in range(R):
            hosted = [e for e in range(E) if x[e, r]]
            for s_idx in range(n_slot):
                for j in range(2):
                    want = params[hosted[s_idx]][j] if s_idx < len(hosted) else torch.zeros(shapes[j], device="cuda", dtype=dtype)
                    assert torch.equal(stacks[r][j][s_idx], want), (r, s_idx, j)
        # backward: every host returns a gradient per slot; owners see the sum over hosts
        grads = [[torch.randn((n_slot,) + s, generator=g, device="cuda").to(dtype) for s in shapes] for _ in range(R)]
        for t in trs:
            t.clear_inbox()
        for r, t in enumerate(trs):
            t.push(grads[r])
        rows = [t.collect() for t in trs]
        torch.cuda.synchronize()
        for e in range(E):
            owner, ls = int(main[e]), e % (E // R)
            for j in range(2):
                want = torch.zeros(shapes[j], device="cuda", dtype=torch.float32)
                for r in range(R):
                    if x[e, r]:
                        hosted = [ee for ee in range(E) if x[ee, r]]
                        want += grads[r][j][hosted.index(e)].float()
                torch.testing.assert_close(rows[owner][j][ls].float(), want, atol=2e-2, rtol=2e-2)
        # the owner-side reduce (hosts stage, owners read with peer loads) gives the same sums
        assert trs[0].owner_reduce_available()
        for r, t in enumerate(trs):
            t.stage(grads[r])
        rows2 = [t.owner_sum() for t in trs]
        torch.cuda.synchronize()
        for r in range(R):
            for j in range(2):
                torch.testing.assert_close(rows2[r][j].float(), rows[r][j].float(), atol=2e-2, rtol=2e-2)
        worlds[0].check_status()
    finally:
        worlds[0].destroy()


def test_module_level_facade_single_rank():
    """``init`` / ``create_tensor`` / ``is_symmetric_tensor`` / ``get`` / ``world_fence`` / ``destroy`` on one rank
    (the calling convention of the reference's ``nccl_gin`` module)."""
    from ep_balance_b200.parallel import onesided

    w = onesided.init(1 << 20, torch.device("cuda", 0))
    try:
        assert onesided.get_rank() == 0 and onesided.get_world_size() == 1
        t = onesided.create_tensor((128, 64), torch.float32)
        assert onesided.is_symmetric_tensor(t) and not onesided.is_symmetric_tensor(torch.zeros(4, device="cuda"))
        t.copy_(torch.arange(128 * 64, device="cuda", dtype=torch.float32).view(128, 64))
        dst = torch.zeros_like(t)
        w.get(dst, t, peer=0)
        w.world_fence(0)              # single rank: nothing to wait for
        w.signal(0, 3, 5)
        w.wait_signal(3, 5)
        torch.cuda.synchronize()
        assert torch.equal(dst, t) and w.test_signal(3) == 5
        w.check_status()
        with pytest.raises(MemoryError):
            onesided.create_tensor((1 << 20,), torch.float32)
    finally:
        onesided.destroy()
    with pytest.raises(RuntimeError):
        onesided.world()
