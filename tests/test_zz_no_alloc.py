"""The allocation-free plan solve, called through its exported C symbol.

Some users of this library cannot call cudaMalloc while it runs: they have given all device
memory to their own pool, or live under a fixed reservation on a shared GPU, or their host
process forbids allocation after start-up.  For them the library exports
``epb_solve_plan_noalloc``, whose scratch memory is a fixed array inside the library.  This test
loads the shared object with ctypes, calls that symbol twice in a row on different inputs (the
second call sees the first call's leftovers in the shared scratch) and requires the outputs to
equal those of the ordinary tensor-level entry point, element for element: the solver is integer
arithmetic, so the tolerance is zero.  Inputs and outputs are the caller's own buffers.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from ep_balance_b200.ops import extension

    extension.load()
    lib = ctypes.CDLL(str(extension._so_path()))
    fn = lib.epb_solve_plan_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int64] + [ctypes.c_int] * 7 + [ctypes.c_void_p] * 4
    lib.epb_noalloc_last_cuda_error.restype = ctypes.c_int
    lib.epb_noalloc_status.restype = ctypes.c_int
    lib.epb_noalloc_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    return lib


def _problem(seed, nodes=2, gpus=4, E=64, extra=2):
    from ep_balance_b200 import EPLBConfig, ProblemSpec, Topology
    from ep_balance_b200.utils.workload import make_loads

    R = nodes * gpus
    loads = make_loads(R, E, 1024, 4, 1.4, 0.25, seed)
    topo = Topology.from_nvlink_rdma(nodes, gpus)
    spec = ProblemSpec.uniform_main_placement(E, R, 3 * 512 * 256 * 2, 512 * 2, E // R + extra)
    return loads, topo, spec, EPLBConfig()


def test_no_alloc_entry_matches_tensor_entry_twice_in_a_row():
    from ep_balance_b200 import Loads, solve

    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    i32 = dict(dtype=torch.int32, device=dev)
    for seed in (21, 22):  # two calls in a row share the library's scratch array
        loads, topo, spec, cfg = _problem(seed)
        R, E = topo.num_ranks, spec.num_experts
        omega = loads.omega.to(**i32).contiguous()
        dom = topo.domain_of_rank.to(**i32).contiguous()
        cost = topo.cost.to(**i32).contiguous()
        main_rank = spec.main_rank.to(**i32).contiguous()
        wbytes = spec.weight_bytes.to(dev).contiguous()
        x = torch.full((E, R), 7, dtype=torch.int8, device=dev)
        q = torch.full((R, E, R), -1, **i32)
        theta = torch.full((1,), -1, dtype=torch.int64, device=dev)
        torch.cuda.synchronize()
        rc = lib.epb_solve_plan_noalloc(omega.data_ptr(), dom.data_ptr(), cost.data_ptr(), main_rank.data_ptr(),
                                        wbytes.data_ptr(), int(spec.s_tok), R, E, topo.num_domains, int(spec.n_slot),
                                        cfg.u_min, cfg.device_stage2_iters, int(cfg.allow_cross_domain),
                                        x.data_ptr(), q.data_ptr(), theta.data_ptr(),
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, (rc, lib.epb_noalloc_last_cuda_error())
        torch.cuda.synchronize()
        want = solve(Loads(loads.omega.to(dev)), topo, spec, cfg)
        assert torch.equal(x, want.x)
        assert torch.equal(q.to(torch.int64), want.q)
        assert int(theta) == int(want.theta)


def _solve_through_c_symbol(lib, dev, loads, topo, spec, cfg, dom_override=None):
    i32 = dict(dtype=torch.int32, device=dev)
    R, E = topo.num_ranks, spec.num_experts
    omega = loads.omega.to(**i32).contiguous()
    dom = (dom_override if dom_override is not None else topo.domain_of_rank).to(**i32).contiguous()
    cost = topo.cost.to(**i32).contiguous()
    main_rank = spec.main_rank.to(**i32).contiguous()
    wbytes = spec.weight_bytes.to(dev).contiguous()
    x = torch.full((E, R), 7, dtype=torch.int8, device=dev)
    q = torch.full((R, E, R), -1, **i32)
    theta = torch.full((1,), -1, dtype=torch.int64, device=dev)
    status = torch.full((4,), -1, **i32)          # the caller's own buffer: nothing is allocated by the library
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    rc = lib.epb_solve_plan_noalloc(omega.data_ptr(), dom.data_ptr(), cost.data_ptr(), main_rank.data_ptr(),
                                    wbytes.data_ptr(), int(spec.s_tok), R, E, topo.num_domains, int(spec.n_slot),
                                    cfg.u_min, cfg.device_stage2_iters, int(cfg.allow_cross_domain),
                                    x.data_ptr(), q.data_ptr(), theta.data_ptr(), stream)
    assert rc == 0, (rc, lib.epb_noalloc_last_cuda_error())
    assert lib.epb_noalloc_status(status.data_ptr(), stream) == 0
    torch.cuda.synchronize(dev)
    return x, q, theta, status.tolist()


def test_no_alloc_entry_on_a_problem_that_needs_the_raised_shared_memory_limit():
    """256 experts on 8 ranks make the solver ask for more than the default 48 KB of dynamic shared memory; the
    limit is raised per device inside the library.  The status word, copied out through the declared call,
    must read zero, and the plan must equal the tensor entry point's."""
    from ep_balance_b200 import Loads, solve

    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    loads, topo, spec, cfg = _problem(31, E=256)
    x, q, theta, status = _solve_through_c_symbol(lib, dev, loads, topo, spec, cfg)
    assert status == [0, 0, 0, 0]
    want = solve(Loads(loads.omega.to(dev)), topo, spec, cfg)
    assert torch.equal(x, want.x) and torch.equal(q.to(torch.int64), want.q) and int(theta) == int(want.theta)


def test_no_alloc_entry_reports_a_domain_id_out_of_range():
    """A rank whose domain id is not in 0..D-1 cannot be solved for; the kernel says so in its status word
    (code 5, bad argument, detail = the rank) instead of returning a plan with that rank's load unset."""
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    loads, topo, spec, cfg = _problem(32)
    bad = topo.domain_of_rank.clone()
    bad[5] = topo.num_domains          # one past the last domain
    _, _, _, status = _solve_through_c_symbol(lib, dev, loads, topo, spec, cfg, dom_override=bad)
    assert status[0] == 5 and status[2] == 5
    # the next, valid call is unaffected (its status word starts at zero again)
    _, _, _, status = _solve_through_c_symbol(lib, dev, loads, topo, spec, cfg)
    assert status == [0, 0, 0, 0]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_no_alloc_entry_on_two_devices_of_one_process():
    """Scratch address and kernel attributes are per device: the same process solves on cuda:0, then on cuda:1."""
    from ep_balance_b200 import Loads, solve

    lib = _lib()
    loads, topo, spec, cfg = _problem(33, E=256)
    for index in (0, 1):
        dev = torch.device("cuda", index)
        with torch.cuda.device(dev):
            x, q, theta, status = _solve_through_c_symbol(lib, dev, loads, topo, spec, cfg)
            want = solve(Loads(loads.omega.to(dev)), topo, spec, cfg)
        assert status == [0, 0, 0, 0]
        assert torch.equal(x, want.x) and torch.equal(q.to(torch.int64), want.q) and int(theta) == int(want.theta)


def test_no_alloc_entry_rejects_sizes_beyond_its_maximum():
    lib = _lib()
    one = torch.zeros(1, dtype=torch.int64, device="cuda").data_ptr()
    args = [one] * 5 + [2]
    too_many_ranks = lib.epb_solve_plan_noalloc(*args, 65, 8, 1, 4, 1, 64, 1, one, one, one, None)
    too_many_experts = lib.epb_solve_plan_noalloc(*args, 8, 1025, 1, 4, 1, 64, 1, one, one, one, None)
    assert too_many_ranks == 1 and too_many_experts == 1
    assert lib.epb_solve_plan_noalloc(*args, 0, 8, 1, 4, 1, 64, 1, one, one, one, None) == 2
