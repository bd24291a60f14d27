"""Plain-loop restatements of the CPU reference functions the reference's own tests embed, used
to pin the numpy oracle. Each cites the test file it restates (paths inside KyleCr4ne/emberlm).
Sizes are tiny, so pure-Python loops are fine."""
import math

import numpy as np

F32 = np.float32


def mm_cpu(a, b, M, K, N, ta, tb):
    """tests/test_bmm.cpp:13-26 (and matmul_cpu, tests/test_matmul.cpp:14-22): float accumulate."""
    a, b = a.reshape(-1), b.reshape(-1)
    c = np.zeros((M, N), dtype=F32)
    for i in range(M):
        for j in range(N):
            acc = F32(0)
            for k in range(K):
                av = a[k * M + i] if ta else a[i * K + k]
                bv = b[j * K + k] if tb else b[k * N + j]
                acc = F32(acc + F32(av * bv))
            c[i, j] = acc
    return c


def rms_norm_cpu(x, w, eps):
    """tests/test_norm.cpp:14-23: fp64 accumulate of x^2, float scale."""
    rows, H = x.shape
    y = np.zeros_like(x)
    for r in range(rows):
        acc = 0.0
        for i in range(H):
            acc += float(x[r, i]) * float(x[r, i])
        scale = F32(1.0) / F32(math.sqrt(F32(F32(acc / H) + F32(eps))))
        for i in range(H):
            y[r, i] = F32(F32(x[r, i] * scale) * w[i])
    return y


def softmax_cpu(x):
    """tests/test_softmax.cpp:14-28."""
    rows, N = x.shape
    y = np.zeros_like(x)
    for r in range(rows):
        m = max(x[r])
        s = 0.0
        for i in range(N):
            y[r, i] = F32(math.exp(F32(x[r, i] - m)))
            s += float(y[r, i])
        inv = F32(1.0 / s)
        for i in range(N):
            y[r, i] = F32(y[r, i] * inv)
    return y


def rope_cpu(x, pos_start, theta):
    """tests/test_rope.cpp:15-32: non-interleaved pairs (i, i+D/2)."""
    B, T, H, D = x.shape
    Dh = D // 2
    y = x.copy()
    for b in range(B):
        for t in range(T):
            for h in range(H):
                for i in range(Dh):
                    inv_freq = F32(math.pow(F32(theta), F32(-(F32(2.0) * i) / F32(D))))
                    ang = F32(F32(pos_start + t) * inv_freq)
                    c, s = F32(math.cos(ang)), F32(math.sin(ang))
                    a0, a1 = x[b, t, h, i], x[b, t, h, i + Dh]
                    y[b, t, h, i] = F32(a0 * c - a1 * s)
                    y[b, t, h, i + Dh] = F32(a0 * s + a1 * c)
    return y


def adamw_closed_form_two_steps(p0=1.0, g=0.1, lr=0.01, b1=0.9, b2=0.999, eps=1e-8):
    """Hand math of tests/test_autograd.cpp:530-573 (constant gradient, two steps, wd = 0)."""
    m1 = (1 - b1) * g
    v1 = (1 - b2) * g * g
    p1 = p0 - lr * ((m1 / (1 - b1)) / (math.sqrt(v1 / (1 - b2)) + eps))
    m2 = b1 * m1 + (1 - b1) * g
    v2 = b2 * v1 + (1 - b2) * g * g
    p2 = p1 - lr * ((m2 / (1 - b1 * b1)) / (math.sqrt(v2 / (1 - b2 * b2)) + eps))
    return p1, p2
