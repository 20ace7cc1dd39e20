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


def test_no_alloc_entry_rejects_sizes_beyond_its_maximum():
    lib = _lib()
    one = torch.zeros(1, dtype=torch.int64, device="cuda").data_ptr()
    args = [one] * 5 + [2]
    too_many_ranks = lib.epb_solve_plan_noalloc(*args, 65, 8, 1, 4, 1, 64, 1, one, one, one, None)
    too_many_experts = lib.epb_solve_plan_noalloc(*args, 8, 1025, 1, 4, 1, 64, 1, one, one, one, None)
    assert too_many_ranks == 1 and too_many_experts == 1
    assert lib.epb_solve_plan_noalloc(*args, 0, 8, 1, 4, 1, 64, 1, one, one, one, None) == 2
