"""GPU: the entry point for callers that may not allocate (sbk_swa_decode_static) against the
ordinary one (sbk_swa_decode), straight through the C ABI.

Some users of this library cannot hand it a scratch buffer: an inference server that spent all
free HBM on its KV pool at start-up, or a control loop that bans allocator calls once it runs.
For them the decode scratch sits in a fixed array inside the library. The array is shared by
every call and remembers what the previous call wrote, so the check runs twice in a row on
different inputs: the second call must not be disturbed by what the first one left behind.
With fixed pieces the order in which a sequence's partials are folded does not depend on timing,
so the two entry points must agree bit for bit (a tolerance here could hide a stale partial); the
CPU oracle is the second, independent comparison, within the bars of the other attention tests.
Collected last on purpose (file name), so a run that stops at the first failure has already
been through every other test.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# same bars as the other attention tests: max-abs 2e-2, mean-rel 1e-3
MAX_ABS, MEAN_REL = 2e-2, 1e-3


def _inputs(seed, lens, H, kvh, D, bs, nb):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    max_blocks = (max(lens) + bs - 1) // bs
    kv = (torch.randn(2, nb, bs, kvh, D, generator=g) / math.sqrt(D)).bfloat16().to(DEV)
    table = torch.stack([torch.randperm(nb, generator=g)[:max_blocks] for _ in range(B)]).to(torch.int32).to(DEV)
    q = (torch.randn(B, H, D, generator=g) / math.sqrt(D)).bfloat16().to(DEV)
    return q, kv, table.contiguous(), torch.tensor(lens, dtype=torch.int32, device=DEV)


def _call(lib, static, q, kv, table, lens, out, lse, H, kvh, D, bs, wl, split, max_pieces, status, ws=None):
    B, nb = q.shape[0], kv.shape[1]
    stream = torch.cuda.current_stream().cuda_stream
    head = (q.data_ptr(), q.stride(0), kv[0].data_ptr(), kv[1].data_ptr(), table.data_ptr(), table.shape[1],
            lens.data_ptr(), B, H, kvh, D, nb, bs, kv.stride(1) * 2, wl, D ** -0.5, out.data_ptr(), 0,
            out.stride(0), lse.data_ptr())
    tail = (split, max_pieces, status.data_ptr(), stream)
    if static:
        return lib.sbk_swa_decode_static(*head, *tail)
    return lib.sbk_swa_decode(*head, ws.data_ptr(), ws.numel(), split, max_pieces, -1, None, None, 0,
                              status.data_ptr(), stream)


def test_static_scratch_entry_point_matches_workspace_entry_point_twice(sb):
    from oracle import ref_ops
    from spikingbrain_7b_b200 import _abi
    lib = _abi.lib
    assert torch.cuda.is_available()
    H, kvh, D, bs, wl, nb = 28, 4, 128, 16, 1023, 400
    split, max_pieces = 8, 9            # several pieces per sequence: the partials in the scratch are used
    assert lib.sbk_swa_static_scratch_bytes() == 16 << 20
    for round_no, (seed, lens) in enumerate([(1, [1100, 17, 640, 2000, 333]), (2, [5, 1500, 1024, 1025, 90])]):
        q, kv, table, lens_t = _inputs(seed, lens, H, kvh, D, bs, nb)
        B = len(lens)
        ws = torch.zeros(lib.sbk_swa_workspace_bytes(B, H, D, max_pieces), dtype=torch.uint8, device=DEV)
        out_ref = torch.empty(B, H, D, dtype=torch.bfloat16, device=DEV)
        out_new = torch.full_like(out_ref, float("nan"))
        lse_ref = torch.empty(B, H, dtype=torch.float32, device=DEV)
        lse_new = torch.full_like(lse_ref, float("nan"))
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        rc = _call(lib, False, q, kv, table, lens_t, out_ref, lse_ref, H, kvh, D, bs, wl, split, max_pieces, status, ws)
        assert rc == 0, lib.sbk_last_error()
        rc = _call(lib, True, q, kv, table, lens_t, out_new, lse_new, H, kvh, D, bs, wl, split, max_pieces, status)
        assert rc == 0, lib.sbk_last_error()
        torch.cuda.synchronize()
        assert status.item() == 0
        assert torch.isfinite(out_new.float()).all(), f"round {round_no}"
        assert torch.equal(out_new, out_ref), f"round {round_no}: the two entry points differ"
        assert torch.equal(lse_new, lse_ref), f"round {round_no}: the two entry points differ in lse"
        want = ref_ops.swa_paged_decode_ref(q.cpu(), kv[0].cpu(), kv[1].cpu(), table.cpu(), lens, wl,
                                            D ** -0.5).bfloat16().float()
        a = out_new.float().cpu()
        assert float((a - want).abs().max()) <= MAX_ABS, f"round {round_no}"
        assert float((a - want).abs().sum() / want.abs().sum()) <= MEAN_REL, f"round {round_no}"


def test_static_scratch_entry_point_rejects_what_does_not_fit(sb):
    from spikingbrain_7b_b200 import _abi
    lib = _abi.lib
    q, kv, table, lens_t = _inputs(3, [64] * 4, 28, 4, 128, 16, 32)
    out = torch.empty(4, 28, 128, dtype=torch.bfloat16, device=DEV)
    lse = torch.empty(4, 28, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # 4 sequences x 400 pieces x 28 heads x 130 floats is more than 16 MiB
    rc = _call(lib, True, q, kv, table, lens_t, out, lse, 28, 4, 128, 16, 63, 1, 400, status)
    assert rc == _abi.SBK_E_WORKSPACE
    msg = lib.sbk_last_error().decode()
    assert "built-in array" in msg and "16777216" in msg
