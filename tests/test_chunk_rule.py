"""The chunked form of the gated delta rule that `dn_chunk_kernel` computes, restated in numpy, against the
token-by-token recurrence of the reference (llm/deltanet.go:365-418): same outputs and same final state.

This checks the algebra the kernel relies on (the A / W matrices, the blocked forward substitution with 16-token
triangles, the decay factors carried across a chunk boundary and a ragged last chunk), not the kernel itself;
the kernel is compared with the oracle in the GPU tests."""
import numpy as np

D, JB, C, BLK = 128, 32, 64, 16


def _inputs(T, seed):
    rng = np.random.default_rng(seed)

    def unit(x):
        return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)

    q, k = unit(rng.standard_normal((T, D))), unit(rng.standard_normal((T, D)))
    v = rng.standard_normal((T, JB))
    g = np.exp(-rng.uniform(0.0, 0.5, T))          # decay per token
    beta = rng.uniform(0.1, 1.0, T)
    s0 = rng.standard_normal((JB, D)) * 0.1        # 32 state rows of one head
    return q, k, v, g, beta, s0


def _sequential(q, k, v, g, beta, s0):
    s, out = s0.copy(), np.zeros((len(g), JB))
    for t in range(len(g)):
        s = s * g[t]
        d = (v[t] - s @ k[t]) * beta[t]
        s = s + np.outer(d, k[t])
        out[t] = s @ q[t]
    return out, s


def _chunked(q, k, v, g, beta, s0):
    T = len(g)
    s, out = s0.copy(), np.zeros((T, JB))
    for c0 in range(0, T, C):
        n = min(C, T - c0)
        K, Q, V = np.zeros((C, D)), np.zeros((C, D)), np.zeros((C, JB))
        G, B = np.ones(C), np.zeros(C)             # past the end: decay 1, beta 0, zero rows
        K[:n], Q[:n], V[:n], G[:n], B[:n] = k[c0:c0 + n], q[c0:c0 + n], v[c0:c0 + n], g[c0:c0 + n], beta[c0:c0 + n]
        L = np.cumsum(np.log(G))
        ratio = np.exp(L[:, None] - L[None, :])
        A = np.tril(B[:, None] * ratio * (K @ K.T), -1)
        W = np.tril(ratio * (Q @ K.T), 0)
        gam = np.exp(L)
        R = B[:, None] * (V - gam[:, None] * (K @ s.T))
        # forward substitution in blocks of 16 tokens: the solved blocks' part comes off the right-hand sides,
        # then the 16 x 16 triangle is solved row by row
        Dm = np.zeros((C, JB))
        for b in range(C // BLK):
            lo = b * BLK
            rhs = R[lo:lo + BLK] - A[lo:lo + BLK, :lo] @ Dm[:lo]
            for tl in range(BLK):
                Dm[lo + tl] = rhs[tl] - A[lo + tl, lo:lo + tl] @ Dm[lo:lo + tl]
        out[c0:c0 + n] = (gam[:, None] * (Q @ s.T) + W @ Dm)[:n]
        s = gam[C - 1] * s + (Dm * np.exp(L[C - 1] - L)[:, None]).T @ K
    return out, s


def test_chunked_rule_is_the_token_by_token_rule():
    for T, seed in ((64, 0), (150, 1), (257, 2), (5, 3)):
        args = _inputs(T, seed)
        o_seq, s_seq = _sequential(*args)
        o_chk, s_chk = _chunked(*args)
        assert np.abs(o_chk - o_seq).max() <= 1e-10 * max(1.0, np.abs(o_seq).max())
        assert np.abs(s_chk - s_seq).max() <= 1e-10 * max(1.0, np.abs(s_seq).max())
