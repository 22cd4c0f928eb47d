"""kbn_moe_permute_static: the permute for callers that cannot allocate device memory (its scratch is
an array inside the library).  Called straight through the C ABI, twice in a row with different
routings, and compared word for word with kbn_moe_permute on the same inputs.  Collected last so that a
failure here cannot hide the result of any other test."""
import pytest
import torch

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _run(lib, check, static, a_q, a_s, ids, e, dev):
    t, k = a_q.shape
    topk = ids.shape[1]
    m_cap = int(lib.kbn_moe_aligned_rows(t, topk, e))
    a_perm = torch.zeros(m_cap, k, dtype=torch.uint8, device=dev)
    s_perm = torch.zeros(m_cap, k // 128, device=dev)
    row_expert = torch.full((m_cap,), -9, dtype=torch.int32, device=dev)
    dest = torch.full((t, topk), -9, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    if static:
        check(lib.kbn_moe_permute_static(a_q.data_ptr(), a_s.data_ptr(), ids.data_ptr(), t, topk, k, e, a_perm.data_ptr(),
                                         s_perm.data_ptr(), row_expert.data_ptr(), dest.data_ptr(), m_cap, stream))
    else:
        ws = torch.empty(int(lib.kbn_moe_permute_workspace_bytes(t, topk, e)), dtype=torch.uint8, device=dev)
        check(lib.kbn_moe_permute(a_q.data_ptr(), a_s.data_ptr(), ids.data_ptr(), t, topk, k, e, a_perm.data_ptr(),
                                  s_perm.data_ptr(), row_expert.data_ptr(), dest.data_ptr(), m_cap, ws.data_ptr(), ws.numel(), stream))
    torch.cuda.synchronize(dev)
    return a_perm.cpu(), s_perm.cpu(), row_expert.cpu(), dest.cpu()


def test_permute_static_matches_permute_on_two_calls_in_a_row(cuda_dev, kbn_lib):
    from kb_nano_b200 import _lib
    gen = torch.Generator().manual_seed(1234)
    for call, (t, topk, e) in enumerate([(300, 8, 64), (77, 2, 5)]):     # second call: other sizes, stale scratch from the first
        k = 512
        a_q = torch.randint(0, 255, (t, k), dtype=torch.uint8, generator=gen).to(cuda_dev)
        a_s = torch.rand(t, k // 128, generator=gen).to(cuda_dev)
        ids = torch.stack([torch.randperm(e, generator=gen)[:topk] for _ in range(t)]).to(torch.int32).to(cuda_dev)
        ref = _run(kbn_lib, _lib.check, False, a_q, a_s, ids, e, cuda_dev)
        got = _run(kbn_lib, _lib.check, True, a_q, a_s, ids, e, cuda_dev)
        for name, r, g in zip(("a_perm", "a_s_perm", "row_expert", "dest_row"), ref, got):
            assert torch.equal(r, g), f"call {call}: {name} differs"          # integer / byte work: exact


def test_permute_static_rejects_sizes_beyond_its_scratch(cuda_dev, kbn_lib):
    x = torch.zeros(16, dtype=torch.uint8, device=cuda_dev)
    p = x.data_ptr()
    rc = kbn_lib.kbn_moe_permute_static(p, p, p, 70000, 1, 128, 4, p, p, p, p, 1 << 20, None)
    assert rc == -3 and b"limit" in kbn_lib.kbn_last_error()
    rc = kbn_lib.kbn_moe_permute_static(p, p, p, 8, 1, 128, 2000, p, p, p, p, 1 << 20, None)
    assert rc == -3
