"""The workspace-free `indexed` entry point (chord_b200_indexed_static_scratch).

Some hosts cannot allocate device memory where they call the GEMM: a serving loop
whose pool is frozen after start-up, or a plugin living in a CUDA context whose
allocator belongs to someone else.  For them the library carries its stream-K scratch
inside its own image.  This test calls that entry point straight through the C ABI and
checks it against the regular entry point (same kernel, so bit-equal), twice in a row
on the shared scratch, and checks that the size limit is enforced.

Collected last on purpose (file name): a failure here cannot hide other tests in a run
that stops at the first failure.  It does not depend on anything they leave behind.
"""

import ctypes

import pytest
import torch

from tests.cases import make_indexed_case

pytestmark = pytest.mark.gpu


def _call(lib, name, device, case, weight, out, locks, workspace=None):
    x = case["x"].to(device)
    sorted_ids = case["sorted_ids"].to(device)
    expert_ids = case["expert_ids"].to(device)
    padded = case["num_tokens_padded"].to(device).reshape(1)
    m = case["topk_ids"].size(0)
    args = [x.data_ptr(), weight.packed.data_ptr(), weight.scale.data_ptr(),
            sorted_ids.data_ptr(), sorted_ids.numel(), expert_ids.data_ptr(), expert_ids.numel(),
            padded.data_ptr(), out.data_ptr(), locks.data_ptr(), locks.numel()]
    if workspace is not None:
        args += [workspace.data_ptr(), workspace.numel() * 4]
    args += [0, m, weight.n, weight.k, weight.num_experts, case["top_k"], case["block_m"],
             torch.cuda.current_stream(device).cuda_stream]
    rc = getattr(lib, name)(*args)
    torch.cuda.synchronize()
    return rc


def test_static_scratch_entry_point_matches_regular_entry_point(device, native_lib):
    import chord_b200
    from chord_b200 import _lib

    # few tiles on 148 SMs: every tile goes through the stream-K scratch
    case = make_indexed_case(num_experts=4, n=256, k=7168, m=12, top_k=2, block_m=16, seed=77)
    weight = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    routes = 12 * 2
    locks = torch.zeros(1024, dtype=torch.int32, device=device)
    ws_bytes = native_lib.chord_b200_gemm_workspace_bytes(16)
    workspace = torch.empty(ws_bytes // 4, dtype=torch.float32, device=device)
    want = torch.full((routes, 256), float("nan"), dtype=torch.bfloat16, device=device)
    assert _call(native_lib, "chord_b200_indexed", device, case, weight, want, locks, workspace) == 0

    before = torch.cuda.memory_allocated(device)
    for attempt in range(2):      # second call runs on the first call's leftovers
        got = torch.full((routes, 256), float("nan"), dtype=torch.bfloat16, device=device)
        rc = _call(native_lib, "chord_b200_indexed_static_scratch", device, case, weight, got, locks)
        assert rc == 0, _lib.last_error()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {attempt}"
        assert bool((locks == 0).all())
        del got
    assert torch.cuda.memory_allocated(device) == before

    # a second shape on the same scratch
    case2 = make_indexed_case(num_experts=8, n=1024, k=512, m=64, top_k=2, block_m=64, seed=78)
    weight2 = chord_b200.pack_w4a16(case2["codes"].to(device), case2["scale"].to(device))
    ws2 = torch.empty(native_lib.chord_b200_gemm_workspace_bytes(64) // 4, dtype=torch.float32,
                      device=device)
    want2 = torch.full((128, 1024), float("nan"), dtype=torch.bfloat16, device=device)
    got2 = torch.full((128, 1024), float("nan"), dtype=torch.bfloat16, device=device)
    assert _call(native_lib, "chord_b200_indexed", device, case2, weight2, want2, locks, ws2) == 0
    assert _call(native_lib, "chord_b200_indexed_static_scratch", device, case2, weight2, got2, locks) == 0
    assert torch.equal(got2.view(torch.int16), want2.view(torch.int16))


def test_static_scratch_entry_point_refuses_large_blocks(device, native_lib):
    import chord_b200
    from chord_b200 import _lib

    case = make_indexed_case(num_experts=2, n=128, k=128, m=40, top_k=2, block_m=128, seed=79)
    weight = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    locks = torch.zeros(1024, dtype=torch.int32, device=device)
    out = torch.zeros((80, 128), dtype=torch.bfloat16, device=device)
    rc = _call(native_lib, "chord_b200_indexed_static_scratch", device, case, weight, out, locks)
    assert rc == 1
    assert "at most 64" in _lib.last_error()
    assert bool((out == 0).all())
