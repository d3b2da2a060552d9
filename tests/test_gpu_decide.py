"""q3_decide_run on the attention runtime (include/q3_decide.h): the reference's
gates for its decision-batch entry point (tests/test_q3_decide.cu:632-821) on
synthetic inputs - B in {1, 2, 4, 8, 16, 32}: zero device allocations and one
host synchronisation in a warm batch, three repeats bit-stable - plus parity of
the logits and of the per-branch decision against the CPU oracle (attention:
src/q3_forward.cu:418-525; head: src/q3_forward.cu:553-607)."""
import numpy as np
import pytest
import torch

import __graft_entry__ as entry
import _cases
import _gpu_harness as harness
import q3_oracle as oracle
import q3_quant_oracle as qo

pytestmark = pytest.mark.gpu
LAYER = 1


@pytest.fixture(scope="module")
def env():
    entry.build()
    pkg = entry.load_package()
    from sera_c_b200 import decide
    return pkg, decide


def _setup(pkg, B, seed=3):
    rng = np.random.default_rng(seed + B)
    lens = [int(x) for x in rng.integers(1, 20, B)]
    case = harness.rounded_case(_cases.Case("decide%d" % B, 70, lens, n_heads=16, n_kv_heads=2,
                                            seed=seed + B, unit_norm_weights=False))
    # prefix prefilled (layer 1), branches acquired; the plan built here is not used
    _, rt, prefix, bset, plan = harness.run_case_native(pkg, case, out_fp32=True,
                                                        return_runtime=True, layer=LAYER)
    plan.close()
    return case, rt, prefix, bset


@pytest.mark.parametrize("B", [1, 2, 4, 8, 16, 32])
def test_decide_run_gates_and_parity(env, B):
    pkg, decide = env
    case, rt, prefix, bset = _setup(pkg, B)
    P, S, H, Hkv, D = case.P, case.S, case.H, case.Hkv, case.D
    width, K, vocab = H * D, 3, 97
    rng = np.random.default_rng(B)
    w = qo.q4k_random_blocks(rng, vocab * (width // 256)).reshape(vocab, -1)
    w_d = torch.from_numpy(w).cuda()
    cands = [rng.choice(vocab, K, replace=False).astype(np.uint32) for _ in range(B)]
    items = [(b, np.arange(n, dtype=np.uint32) + 11, cands[b])
             for b, n in enumerate(case.branch_lens)]
    g = torch.Generator().manual_seed(B)
    mk = lambda a: harness.dev(a, torch.bfloat16)
    # layer 0: unrelated activations (its prefix KV is empty: zeros); layer 1: the case
    q = [torch.randn(S, H, D, generator=g).to(torch.bfloat16).cuda(), mk(case.q[P:])]
    k = [torch.randn(S, Hkv, D, generator=g).to(torch.bfloat16).cuda(), mk(case.k[P:])]
    v = [torch.randn(S, Hkv, D, generator=g).to(torch.bfloat16).cuda(), mk(case.v[P:])]
    out = [torch.zeros(S, H, D, dtype=torch.float32, device="cuda") for _ in range(2)]
    hidden = out[1].view(S, width)              # stand-in for the rest of the model
    calls = []

    def hook(user, layer, ids, tokens, stream):
        calls.append((layer, tokens, ids[0], ids[tokens - 1]))
        return True

    torch.cuda.synchronize()
    first = None
    for rep in range(4):
        res, st = decide.decide_run(rt, prefix, bset, items, q, k, v, out, hidden, w_d, 12,
                                    vocab, hook=hook)
        if rep == 0:
            first = res                          # cold: may grow the staging buffers
            continue
        assert st.cuda_allocations == 0 and st.cuda_frees == 0          # warm batch
        assert st.host_syncs == 1                # the boundary synchronisation only
        assert st.kernel_launches_per_batch == 2 * 2 + 1
        assert st.batch == B and st.suffix_tokens_total == S
        assert st.suffix_forward_ms > 0 and st.candidate_head_ms > 0
        for a, b in zip(res, first):             # repeatable bit for bit
            assert a[0] == b[0] and np.array_equal(a[1], b[1])
    assert len(calls) == 8 and calls[0][:2] == (0, S) and calls[1][0] == 1
    assert calls[0][2] == 11 and calls[0][3] == 11 + case.branch_lens[-1] - 1
    assert rt.stats().device_status == 0

    # parity: attention rows of the last layer, then the head, through the oracle
    ref = oracle.run_case(case)["out"][P:].reshape(S, width)
    assert np.abs(out[1].cpu().numpy().reshape(S, width) - ref).max() <= 2e-3
    offs = case.branch_offsets.astype(np.int32)
    ids = np.concatenate(cands).astype(np.int32)
    want = qo.candidate_logits_batched(qo.gather_last_rows(ref, offs), w, 12, ids, K)
    want = want.reshape(B, K)
    for b, (pred, logits, probs) in enumerate(first):
        assert np.abs(logits - want[b]).max() <= 2e-3 * np.abs(want).max()
        assert pred == int(want[b].argmax())
        e = np.exp(want[b] - want[b].max())
        assert np.abs(probs - e / e.sum()).max() < 5e-3 and abs(probs.sum() - 1) < 1e-5
    bset.close()
    prefix.close()
    rt.close()


def test_decide_run_refusals(env):
    pkg, decide = env
    case, rt, prefix, bset = _setup(pkg, 2)
    S, H, Hkv, D = case.S, case.H, case.Hkv, case.D
    z = lambda h, dt=torch.bfloat16: [torch.zeros(S, h, D, dtype=dt, device="cuda")]
    out = z(H, torch.float32)
    w = torch.zeros(8, (H * D // 256) * 144, dtype=torch.uint8, device="cuda")
    run = lambda items: decide.decide_run(rt, prefix, bset, items, z(H), z(Hkv), z(Hkv), out,
                                          out[0].view(S, -1), w, 12, 8)
    tok = np.arange(3, dtype=np.uint32)
    with pytest.raises(pkg.Q3Error, match="bad branch count"):
        run([(0, tok, [1, 2])] * 3)                       # the set holds 2 branches
    with pytest.raises(pkg.Q3Error, match="bad candidate count"):
        run([(0, tok, list(range(31)))])
    with pytest.raises(pkg.Q3Error, match="invalid decision item"):
        run([(0, tok, [1, 2]), (1, tok, [1])])            # candidate counts differ
    with pytest.raises(pkg.Q3Error, match="invalid decision item"):
        run([(0, np.arange(64, dtype=np.uint32), [1, 2])])  # longer than max_suffix
    with pytest.raises(pkg.Q3Error, match="invalid branch handle"):
        run([(5, tok, [1, 2])])
    bset.close()
    prefix.close()
    rt.close()
