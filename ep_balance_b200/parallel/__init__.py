"""Expert-parallel runtime pieces.

  symm.py           symmetric heap (one allocation per rank, mapped into every peer)
  onesided.py       symmetric tensors, batched get/put, signals, fences over that heap
  symm_weights.py   device-initiated replica weight channel built on onesided.py
  omega.py          load-matrix collection for the portable path
  rebalancer.py     gather -> solve -> materialise orchestration, plan ring
  hooks.py          weight materialiser / dispatcher protocols
  comm.py           autograd-aware collectives
  physical.py       unit -> physical instance routing on host tensors
  grouped_mlp.py    grouped / padded expert MLP callbacks
  library_path.py   portable apply path (gloo / NCCL): ragged and zero-sync padded token transports
  overlap.py        comm / weight lanes of the portable path, weight lease, prefetch on backward
  transport_model.py  host model of the fused layer's transport (buffer layout, items, arrival signals)
  health.py         host-side failure detection (heartbeats, step guard)
"""
