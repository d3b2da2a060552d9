"""Seeded synthetic inputs shared by the golden-vector generator, the CPU tests
and the GPU parity tests.

A case is one layer of the Qwen3-32B attention geometry: a shared prefix of P
tokens followed by B packed suffix branches, rows laid out
[prefix tokens | branch 0 tokens | branch 1 tokens | ...]. Prefix token i sits
at position i; token j of every branch sits at position P + j (the reference
packs them this way, src/q3_decide.cu:440-464).
"""
import hashlib

import numpy as np
import torch


class Case:
    def __init__(self, name, prefix_len, branch_lens, n_heads=64, n_kv_heads=8,
                 head_dim=128, seed=0, unit_norm_weights=True, theta=1e6,
                 eps=1e-6, branch_handles=None, golden_rows=None,
                 golden_heads=None):
        self.name = name
        self.P = int(prefix_len)
        self.branch_lens = [int(x) for x in branch_lens]
        self.H, self.Hkv, self.D = n_heads, n_kv_heads, head_dim
        self.theta, self.eps = float(theta), float(eps)
        self.scale = np.float32(1.0 / np.sqrt(head_dim))
        self.S = int(sum(self.branch_lens))
        self.T = self.P + self.S
        g = torch.Generator().manual_seed(seed)
        self.q = torch.randn(self.T, n_heads, head_dim, generator=g).numpy()
        self.k = torch.randn(self.T, n_kv_heads, head_dim, generator=g).numpy()
        self.v = torch.randn(self.T, n_kv_heads, head_dim, generator=g).numpy()
        if unit_norm_weights:
            self.q_norm_w = np.ones(head_dim, np.float32)
            self.k_norm_w = np.ones(head_dim, np.float32)
        else:
            self.q_norm_w = (0.5 + torch.rand(head_dim, generator=g)).numpy()
            self.k_norm_w = (0.5 + torch.rand(head_dim, generator=g)).numpy()
        B = len(self.branch_lens)
        self.branch_handles = (list(range(B)) if branch_handles is None
                               else list(branch_handles))
        pos = list(range(self.P))
        tb, tl, off = [], [], [0]
        for b, n in enumerate(self.branch_lens):
            pos += [self.P + j for j in range(n)]
            tb += [self.branch_handles[b]] * n
            tl += list(range(n))
            off.append(off[-1] + n)
        self.positions = np.asarray(pos, np.uint32)
        self.token_branch = np.asarray(tb, np.uint32)      # suffix rows only
        self.token_local_pos = np.asarray(tl, np.uint32)   # suffix rows only
        self.branch_offsets = np.asarray(off, np.uint32)
        self.golden_rows = golden_rows if golden_rows is not None else list(range(self.T))
        self.golden_heads = golden_heads if golden_heads is not None else list(range(n_heads))

    @property
    def mask(self):
        """[T, T] bool: True where query row i may attend to key row j."""
        m = np.zeros((self.T, self.T), bool)
        P = self.P
        m[:P, :P] = np.tril(np.ones((P, P), bool))
        r = P
        for n in self.branch_lens:
            m[r:r + n, :P] = True
            m[r:r + n, r:r + n] = np.tril(np.ones((n, n), bool))
            r += n
        return m

    def input_sha256(self):
        h = hashlib.sha256()
        for a in (self.q, self.k, self.v, self.q_norm_w, self.k_norm_w):
            h.update(np.ascontiguousarray(a, np.float32).tobytes())
        return h.hexdigest()


# name -> constructor arguments. "config1" is the CPU-runnable configuration
# of the benchmark definition (256-token prefix + 3 branches x 8 tokens).
_SPECS = {
    "config1": dict(prefix_len=256, branch_lens=[8, 8, 8], seed=0,
                    golden_rows=[0, 1, 15, 16, 127, 255, 256, 263, 264, 270, 272, 279],
                    golden_heads=[0, 7, 8, 21, 37, 63]),
    "ragged": dict(prefix_len=19, branch_lens=[5, 3, 1, 18], n_heads=16,
                   n_kv_heads=2, seed=7, unit_norm_weights=False,
                   branch_handles=[2, 0, 3, 1], golden_heads=[0, 5, 8, 15]),
    "prefill_only": dict(prefix_len=45, branch_lens=[], n_heads=8, n_kv_heads=1,
                         seed=3, unit_norm_weights=False, golden_heads=[0, 3, 7]),
}
GOLDEN_CASES = ["config1", "ragged", "prefill_only"]


def make_case(name):
    return Case(name, **_SPECS[name])
