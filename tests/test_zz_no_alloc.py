"""The allocation-free decode entry point (ahpc_paged_decode_static) against the regular one.

This file sorts last on purpose: if it fails, a run that stops at the first failure has already
run every other test.

Who the entry point is for: callers that cannot call cudaMalloc at decode time - a server that gave
all device memory to its own arena and forbids driver allocations afterwards, or code inside a
region its framework declares allocation-free.  Its split-KV scratch is a fixed array inside the
library image, shared by every call on the device and never cleared, so the checks below make two
calls in a row with different shapes: the second call must not be disturbed by what the first left
behind, and both must equal what ahpc_paged_decode returns for the same arguments.
"""
import numpy as np
import pytest
import torch

from attention_b200 import abi, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2          # the tolerance of the FP16/BF16 decode tests


def _filled_pool(lens, heads=4, head_dim=128, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    pages = sum((n + 15) // 16 for n in lens) + 4
    pool = ops.KVPool(num_pages=pages, heads=heads, head_dim=head_dim, dtype=torch.float16, max_seqs=len(lens),
                      max_pages_per_seq=max((n + 15) // 16 for n in lens) + 1)
    seqs = []
    for n in lens:
        s = pool.seq_create()
        k = torch.randn((n, heads, head_dim), generator=g, device=DEV).half()
        v = torch.randn((n, heads, head_dim), generator=g, device=DEV).half()
        pool.append([s], [n], k, v)
        seqs.append(s)
    return pool, seqs, g


def test_static_decode_matches_regular_decode_on_two_calls_in_a_row():
    pool, seqs, g = _filled_pool([1, 17, 700, 2500, 64])
    # first call: all sequences, library-chosen split
    q1 = torch.randn((len(seqs), 4, 128), generator=g, device=DEV).half()
    want1 = pool.decode(seqs, q1)
    got1 = pool.decode(seqs, q1, no_alloc=True)
    torch.cuda.synchronize()
    assert float((got1.float() - want1.float()).abs().max()) <= TOL
    # second call straight after: other sequences, other split, other query type - the array still holds call one's partials
    order = [seqs[3], seqs[1], seqs[3]]
    q2 = torch.randn((3, 4, 128), generator=g, device=DEV).to(torch.bfloat16)
    q2[2] = q2[0]                                         # the same sequence asked the same question twice
    want2 = pool.decode(order, q2, split_tokens=128)
    got2 = pool.decode(order, q2, split_tokens=128, no_alloc=True)
    torch.cuda.synchronize()
    assert float((got2.float() - want2.float()).abs().max()) <= TOL
    assert torch.equal(got2[0], got2[2])
    # and once more with the first arguments: same answer as before
    again = pool.decode(seqs, q1, no_alloc=True)
    assert torch.equal(again, got1)
    assert np.isfinite(again.float().cpu().numpy()).all()
    pool.close()


def test_static_decode_refuses_what_does_not_fit_and_host_tensors():
    cap = abi.lib().ahpc_paged_decode_static_capacity()
    assert cap == 32 * 1024 * 1024
    pool, seqs, g = _filled_pool([4096], heads=32)
    q = torch.randn((1, 32, 128), generator=g, device=DEV).half()
    many = seqs * 4096                                   # 4096 x 256 chunks x 32 heads of partials: far beyond the array
    qq = q.expand(4096, 32, 128).contiguous()
    with pytest.raises(abi.AhpcError) as e:
        pool.decode(many, qq, split_tokens=16, no_alloc=True)
    assert e.value.status == 3 and "built-in" in str(e.value)
    with pytest.raises(abi.AhpcError) as e:              # host tensors would need a staging allocation
        pool.decode(seqs, q.cpu(), no_alloc=True)
    assert e.value.status == 1
    out = pool.decode(seqs, q, no_alloc=True)            # the pool still works after the refusals
    assert float((out.float() - pool.decode(seqs, q).float()).abs().max()) <= TOL
    pool.close()
