"""The oracle's restatement of Sampler::sample (wick/src/sampler.rs:64-158, uniform draw supplied by the caller) against
a second, plain-numpy restatement of the same source lines, and against closed-form cases."""
import numpy as np

F32 = np.float32


def numpy_sample(orc, logits, temperature, top_k, top_p, r):
    l = np.array(logits, F32)
    n = l.size
    if temperature <= 0 or top_k == 1:
        return orc.argmax(l)
    l = (l * (F32(1.0) / F32(temperature))).astype(F32)
    if 0 < top_k < n:
        thr = np.sort(l)[::-1][top_k - 1]
        l[l < thr] = -np.inf
    if top_p < 1.0:
        idx = [i for i in range(n) if np.isfinite(l[i])]
        idx.sort(key=lambda i: (-float(l[i]), i))
        if idx:
            mx = l[idx[0]]
            probs = [F32(np.exp(F32(l[i] - mx))) for i in idx]
            s = F32(0)
            for p in probs:
                s = F32(s + p)
            cum, cut = F32(0), len(idx)
            for j, p in enumerate(probs):
                cum = F32(cum + F32(p / s))
                if cum >= F32(top_p):
                    cut = j + 1
                    break
            for i in idx[cut:]:
                l[i] = -np.inf
    p = orc.softmax(l) if hasattr(orc, "softmax") else None
    if p is None:
        mx = l.max()
        e = orc.expf((l - mx).astype(F32))
        p = (e * F32(1.0 / float(np.sum(e.astype(np.float64))))).astype(F32)
    cum = F32(0)
    for i in range(n):
        cum = F32(cum + p[i])
        if cum >= F32(r):
            return i
    return n - 1


def test_sampler_matches_numpy_restatement(orc):
    rng = np.random.default_rng(0)
    for case in range(60):
        n = int(rng.integers(2, 400))
        logits = (rng.standard_normal(n) * rng.uniform(0.5, 6)).astype(F32)
        if case % 7 == 0:
            logits[rng.integers(0, n, size=3)] = logits.max()       # ties at the top
        temperature = float(rng.choice([0.0, 0.3, 0.7, 1.0, 1.5]))
        top_k = int(rng.choice([0, 1, 2, 5, 40, n, n + 5]))
        top_p = float(rng.choice([0.1, 0.5, 0.9, 0.95, 1.0]))
        r = float(F32(rng.random()))
        assert orc.sample(logits, temperature, top_k, top_p, r) == numpy_sample(orc, logits, temperature, top_k, top_p, r), \
            (case, n, temperature, top_k, top_p, r)


def test_sampler_closed_form_cases(orc):
    logits = np.array([0.0, 1.0, 2.0, 3.0], F32)
    assert orc.sample(logits, 0.0, 40, 0.9, 0.5) == 3          # temperature 0: argmax
    assert orc.sample(logits, 0.7, 1, 0.9, 0.5) == 3           # top_k 1: argmax
    assert orc.sample(logits, 1.0, 0, 1.0, 0.0) == 0           # r = 0 stops at element 0
    assert orc.sample(logits, 1.0, 0, 1.0, 0.9999999) == 3
    # softmax [0.0321, 0.0871, 0.2369, 0.6439]: cumulative 0.0321, 0.1192, 0.3561, 1.0
    assert orc.sample(logits, 1.0, 0, 1.0, 0.10) == 1
    assert orc.sample(logits, 1.0, 0, 1.0, 0.30) == 2
    assert orc.sample(logits, 1.0, 2, 1.0, 0.10) == 2          # top-2 keeps {2, 3}: probabilities 0.269, 0.731
    assert orc.sample(logits, 1.0, 0, 0.5, 0.99) == 3          # nucleus 0.5: only the top token survives
