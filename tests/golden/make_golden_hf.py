"""Generate golden vectors for the attention path from the HuggingFace Qwen3
functions that the reference's Python oracle runs.

The reference's tools/qwen3_q4_oracle.py:88-92,151-154 builds a HuggingFace
Qwen3ForCausalLM with attn_implementation="sdpa"; the attention arithmetic it
executes is transformers.models.qwen3.modeling_qwen3 (Qwen3RMSNorm,
Qwen3RotaryEmbedding, apply_rotary_pos_emb, repeat_kv) plus
torch.nn.functional.scaled_dot_product_attention. This script calls exactly
those functions on CPU in fp32 on seeded synthetic q/k/v, with an explicit
[shared prefix | own causal suffix] mask, and stores a subset of the results.

Run from the repository root (CPU only, about half a minute):

    python tests/golden/make_golden_hf.py

Outputs tests/golden/hf_case_*.npz. The inputs are NOT stored; they are
regenerated from the seed by tests/_cases.py and their SHA-256 is stored so a
changed generator is detected instead of silently compared.
"""
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import _cases  # noqa: E402  (tests/_cases.py)


def hf_attention(case):
    from transformers.models.qwen3 import modeling_qwen3 as m
    from transformers.models.qwen3.configuration_qwen3 import Qwen3Config

    q, k, v = (torch.from_numpy(a) for a in (case.q, case.k, case.v))
    T, H, D = q.shape
    Hkv = k.shape[1]
    cfg = Qwen3Config(hidden_size=H * D, num_attention_heads=H,
                      num_key_value_heads=Hkv, head_dim=D,
                      rope_theta=case.theta, max_position_embeddings=1 << 17,
                      num_hidden_layers=1, intermediate_size=64, vocab_size=16)
    qn = m.Qwen3RMSNorm(D, eps=case.eps)
    kn = m.Qwen3RMSNorm(D, eps=case.eps)
    with torch.no_grad():
        qn.weight.copy_(torch.from_numpy(case.q_norm_w))
        kn.weight.copy_(torch.from_numpy(case.k_norm_w))
        rot = m.Qwen3RotaryEmbedding(cfg)
        pos = torch.from_numpy(case.positions.astype(np.int64))[None, :]
        # [1, heads, T, D] as in Qwen3Attention.forward
        qs = qn(q[None]).transpose(1, 2)
        ks = kn(k[None]).transpose(1, 2)
        vs = v[None].transpose(1, 2)
        cos, sin = rot(vs, pos)
        qs, ks = m.apply_rotary_pos_emb(qs, ks, cos, sin)
        mask = torch.from_numpy(case.mask)[None, None]
        out = torch.nn.functional.scaled_dot_product_attention(
            qs, m.repeat_kv(ks, H // Hkv), m.repeat_kv(vs, H // Hkv),
            attn_mask=mask, scale=float(case.scale))
    return (qs.transpose(1, 2)[0].numpy(), ks.transpose(1, 2)[0].numpy(),
            out.transpose(1, 2)[0].contiguous().numpy())


def main():
    import transformers
    for name in _cases.GOLDEN_CASES:
        case = _cases.make_case(name)
        q2, k2, out = hf_attention(case)
        rows = np.asarray(case.golden_rows, dtype=np.int64)
        heads = np.asarray(case.golden_heads, dtype=np.int64)
        kvh = np.unique(heads // (case.q.shape[1] // case.k.shape[1]))
        path = os.path.join(HERE, "hf_case_%s.npz" % name)
        np.savez(path,
                 rows=rows, heads=heads, kv_heads=kvh,
                 q2=q2[rows][:, heads], k2=k2[rows][:, kvh],
                 out=out[rows][:, heads],
                 input_sha256=np.array(case.input_sha256()),
                 versions=np.array("torch %s transformers %s" % (
                     torch.__version__, transformers.__version__)))
        print(name, "->", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
