"""GPU parity tests of the last-row gather and the selected-row LM head
(include/q3_lmhead.h) against the CPU oracle: logits within 1e-4 of the
double-precision dot (relative to the largest logit), identical argmax per
branch, for Q4_K and Q6_K output weights."""
import numpy as np
import pytest
import torch

import __graft_entry__ as entry
import q3_quant_oracle as qo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def head():
    entry.build()
    entry.load_package()
    from sera_c_b200 import lmhead
    return lmhead


def _weight(rng, qtype, vocab, hidden):
    nb = vocab * (hidden // 256)
    if qtype == 12:
        return qo.q4k_random_blocks(rng, nb).reshape(vocab, -1)
    return qo.q6k_random_blocks(rng, nb).reshape(vocab, -1)


@pytest.mark.parametrize("qtype", [12, 14])
@pytest.mark.parametrize("lens,K,hidden", [([3, 1, 7, 2], 3, 512), ([16] * 32, 3, 5120),
                                           ([5, 9], 11, 1024)])
def test_gather_and_logits_match_oracle(head, qtype, lens, K, hidden):
    rng = np.random.default_rng(qtype * 100 + K + hidden)
    vocab = 300
    w = _weight(rng, qtype, vocab, hidden)
    T, B = sum(lens), len(lens)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    rows = rng.standard_normal((T, hidden)).astype(np.float32)
    ids = rng.integers(0, vocab, B * K).astype(np.int32)
    rows_d = torch.from_numpy(rows).cuda()
    offs_d = torch.from_numpy(offs).cuda()
    ids_d = torch.from_numpy(ids).cuda()
    w_d = torch.from_numpy(w).cuda()

    last = head.gather_last_rows(rows_d, offs_d)
    assert np.array_equal(last.cpu().numpy(), qo.gather_last_rows(rows, offs))
    want = qo.candidate_logits_batched(qo.gather_last_rows(rows, offs), w, qtype, ids, K)
    tol = 1e-4 * np.abs(want).max()
    got = head.candidate_logits_batched(last, w_d, qtype, vocab, ids_d, K).cpu().numpy()
    assert np.abs(got - want).max() < tol
    fused, best = head.candidate_head(rows_d, offs_d, w_d, qtype, vocab, ids_d, K)
    torch.cuda.synchronize()
    assert np.array_equal(fused.cpu().numpy(), got)             # same kernel, same order
    assert np.array_equal(best.cpu().numpy(), want.reshape(B, K).argmax(axis=1))


def test_bad_candidate_and_arguments(head):
    from sera_c_b200 import Q3Error
    rng = np.random.default_rng(0)
    w = torch.from_numpy(_weight(rng, 12, 10, 256)).cuda()
    h = torch.zeros(1, 256, dtype=torch.float32, device="cuda")
    ids = torch.tensor([3, 10], dtype=torch.int32, device="cuda")     # 10 is out of range
    out = head.candidate_logits_batched(h, w, 12, 10, ids, 2).cpu().numpy()
    assert out[0] == 0.0 and np.isnan(out[1])
    with pytest.raises(Q3Error, match="neither Q4_K nor Q6_K"):
        head.candidate_logits_batched(h, w, 2, 10, ids, 2)
    with pytest.raises(Q3Error, match="invalid argument"):
        head.candidate_logits_batched(torch.zeros(1, 100, device="cuda"), w, 12, 10, ids, 2)


@pytest.mark.parametrize("name", ["config1", "ragged"])
def test_argmax_identical_through_the_candidate_head(head, name):
    """The path's own consumer: the attention rows of the packed suffix (GPU,
    fp32 output) go through q3_cuda_candidate_head with a Q6_K weight whose
    row length is the attention width; the per-branch decision must equal the
    one the oracle reaches from the oracle's attention rows."""
    import _cases
    import _gpu_harness as harness
    import q3_oracle as oracle
    pkg = entry.load_package()
    case = harness.rounded_case(_cases.make_case(name))
    ref = oracle.run_case(case)["out"]                     # [T, H, D]
    got = harness.run_case_native(pkg, case, out_fp32=True)
    P, S, width, K = case.P, case.S, case.H * case.D, 5
    vocab = 64
    rng = np.random.default_rng(17)
    w = qo.q6k_random_blocks(rng, vocab * (width // 256)).reshape(vocab, -1)
    B = len(case.branch_lens)
    ids = rng.integers(0, vocab, B * K).astype(np.int32)
    offs = case.branch_offsets.astype(np.int32)            # offsets inside the suffix
    rows = torch.from_numpy(np.ascontiguousarray(got[P:].reshape(S, width))).cuda()
    logits, best = head.candidate_head(rows, torch.from_numpy(offs).cuda(),
                                       torch.from_numpy(w).cuda(), 14, vocab,
                                       torch.from_numpy(ids).cuda(), K)
    torch.cuda.synchronize()
    want = qo.candidate_logits_batched(
        qo.gather_last_rows(ref[P:].reshape(S, width), offs), w, 14, ids, K).reshape(B, K)
    assert np.array_equal(best.cpu().numpy(), want.argmax(axis=1))
    assert np.abs(logits.cpu().numpy().reshape(B, K) - want).max() < 2e-3 * np.abs(want).max()
