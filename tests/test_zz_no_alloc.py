"""The sort-and-pad entry point for callers that cannot allocate device memory.

Some hosts of the library may not call cudaMalloc while they run: a serving
process whose own pool already owns all of HBM has nothing left to hand out,
and a decode loop with a latency budget cannot take the device-wide stall an
allocation causes.  ``mb200_align_noalloc`` keeps its scratch in a fixed array
inside the library, so such a caller passes only inputs and preallocated
outputs.  This test drives it through the C ABI and requires bit-identical
results to ``mb200_align`` (the integer stages have no tolerance), on
back-to-back calls whose scratch footprints differ, so that anything the first
call left in the shared array would show up in the second.

The file name makes pytest collect it last: a run that stops at the first
failure has then already executed every other test.
"""

import numpy as np
import pytest
import torch

from moe_bench_b200 import capi
from moe_bench_b200 import problem as P
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _routing(dist, tokens, experts, topk, seed):
    cfg = P.MoEBenchConfig(
        hidden_size=256, intermediate_size=128, num_experts=experts, topk=topk, world_size=1,
        routing=P.RoutingConfig(distribution=P.Distribution(dist)), seed=seed, device="cpu",
    )
    return P._make_routing(cfg, tokens, torch.Generator().manual_seed(seed + 99))[0].to(DEV)


def _same(a, b):
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_noalloc_align_matches_align_on_consecutive_calls():
    # 1) large: three-kernel path, fills many unit histograms of the shared array
    # 2) small, fewer experts: one-block path, reads a different part of the same array
    # 3) expert-parallel map with empty experts, again after a larger call
    cases = [
        ("uniform", 8192, 256, 8, None),
        ("skewed", 100, 64, 4, None),
        ("uniform", 3000, 256, 8, 8),
        ("single", 1, 256, 8, None),
    ]
    for i, (dist, tokens, experts, topk, ep) in enumerate(cases):
        ids = _routing(dist, tokens, experts, topk, seed=i)
        emap, local = None, experts
        if ep:
            local = experts // ep
            emap = torch.full((experts,), -1, dtype=torch.int32, device=DEV)
            emap[5 * local : 6 * local] = torch.arange(local, dtype=torch.int32, device=DEV)
        pad = (16, 128)[i % 2]  # both padding granules the library uses
        want = capi.align(ids, emap, local, pad)
        # preallocated outputs: from here on the call itself allocates nothing
        cap = capi.row_capacity(tokens, topk, local, pad)
        outs = (
            torch.empty(local, dtype=torch.int32, device=DEV),
            torch.empty(local + 1, dtype=torch.int32, device=DEV),
            torch.full((cap,), -2, dtype=torch.int32, device=DEV),
            torch.empty(tokens * topk, dtype=torch.int32, device=DEV),
        )
        outs2 = tuple(t.clone() for t in outs)
        if i == 0:
            # first call on the device: looks up the built-in array's address
            capi.align_noalloc(ids, emap, local, outputs=tuple(t.clone() for t in outs), pad_rows=pad)
        torch.cuda.synchronize()
        held_by_torch = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        got = capi.align_noalloc(ids, emap, local, outputs=outs, pad_rows=pad)
        got_again = capi.align_noalloc(ids, emap, local, outputs=outs2, pad_rows=pad)
        torch.cuda.synchronize()
        # neither torch nor the library took device memory during the two calls
        assert torch.cuda.memory_allocated() == held_by_torch
        assert torch.cuda.mem_get_info()[0] >= free_before
        _same(got, want)
        _same(got_again, want)
        # and against the CPU oracle directly, not only through the other entry point
        o_counts, o_off, o_sorted, o_inv = O.align(ids.cpu().numpy(), None if emap is None else emap.cpu().numpy(),
                                                   local, pad)
        assert np.array_equal(got[0].cpu().numpy(), o_counts) and np.array_equal(got[1].cpu().numpy() * pad, o_off)
        used = int(o_off[-1])
        assert np.array_equal(got[2].cpu().numpy()[:used], o_sorted) and np.array_equal(got[3].cpu().numpy(), o_inv)
        # drop this iteration's tensors now, so the next iteration's measurement sees no frees
        del got, got_again, want, outs, outs2


def test_noalloc_align_refuses_oversized_problems():
    lib = capi.load()
    ids = torch.zeros(4, 2, dtype=torch.int32, device=DEV)
    out = torch.empty(4096, dtype=torch.int32, device=DEV)
    p = ids.data_ptr()
    o = out.data_ptr()
    # too many local experts
    rc = lib.mb200_align_noalloc(p, 4, 2, None, 257, o, o, o, o, 4096, 16, None)
    assert rc == 5 and b"at most 256" in lib.mb200_last_error()
    # too many assignments (nothing is launched, so the pointers are never used)
    rc = lib.mb200_align_noalloc(p, (1 << 20) // 2 + 1, 2, None, 8, o, o, o, o, 1 << 30, 16, None)
    assert rc == 5 and b"mb200_align" in lib.mb200_last_error()
    with pytest.raises(capi.MB200Error):
        capi.align_noalloc(torch.zeros(4, 2, dtype=torch.int32, device=DEV), None, 300)
