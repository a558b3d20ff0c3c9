"""GPU tests of `caten_b200_sample` (temperature / top-k sampling; beyond the reference, whose
generate loop is greedy): the kernel's choice against a float64 numpy statement of the same rule,
with the uniform numbers chosen away from the boundaries of the cumulative distribution."""
import numpy as np
import pytest

from caten_b200 import synthetic as S
from caten_b200.gpt2 import GPT2, gpt2_generate

pytestmark = pytest.mark.gpu


def reference_choice(x, u, temperature, top_k):
    """(index, distance of u*Z to the nearest CDF boundary relative to Z)"""
    x = x.astype(np.float64)
    V = x.size
    keep = np.ones(V, bool) if top_k <= 0 or top_k >= V else x >= np.sort(x)[V - top_k]
    w = np.where(keep, np.exp((x - x.max()) / temperature), 0.0)
    cdf = np.cumsum(w)
    target = u * cdf[-1]
    i = int(np.searchsorted(cdf, target, side="left"))
    while w[i] == 0.0:
        i += 1
    return i, np.abs(cdf - target).min() / cdf[-1]


@pytest.mark.parametrize("V,temperature,top_k", [(50257, 1.0, 0), (50257, 0.7, 40), (1003, 1.3, 5), (4099, 0.5, 1), (257, 2.0, 300)])
def test_sample_matches_the_stated_rule(rt, V, temperature, top_k):
    rng = np.random.Generator(np.random.PCG64(V + top_k))
    rows = 48
    logits = (rng.standard_normal((rows, V), dtype=np.float32) * 3).astype(np.float32)
    logits[3, 10:14] = logits[3].max()          # ties at the top
    u = np.empty(rows, np.float32)
    want = np.empty(rows, np.int64)
    for r in range(rows):
        for _ in range(100):                    # a uniform number that is not within rounding of a boundary
            cand = np.float32(rng.random())
            i, margin = reference_choice(logits[r], float(cand), temperature, top_k)
            if margin > 1e-4:
                break
        u[r], want[r] = cand, i
    got = rt.sample(rt.transfer_from_array(logits), u, temperature, top_k).numpy()
    np.testing.assert_array_equal(got, want)
    if top_k == 1:  # the single most likely id, except in the row where several ids tie for it
        rest = np.arange(rows) != 3
        np.testing.assert_array_equal(got[rest], logits.argmax(1)[rest])


def test_zero_temperature_is_argmax_and_u_zero_is_first_kept(rt):
    rng = np.random.Generator(np.random.PCG64(1))
    logits = rng.standard_normal((7, 1000), dtype=np.float32)
    d = rt.transfer_from_array(logits)
    np.testing.assert_array_equal(rt.sample(d, np.zeros(7, np.float32), 0.0, 0).numpy(), logits.argmax(1))
    got = rt.sample(d, np.zeros(7, np.float32), 1.0, 3).numpy()
    top3 = np.argsort(-logits, 1)[:, :3]
    np.testing.assert_array_equal(got, top3.min(1))   # u = 0: the lowest index among the kept three


def test_generate_with_sampling_is_seeded_and_stays_in_the_top_k(rt):
    p = S.GPT2Params(n_layers=2, n_heads=2, dim=128, vocab_size=1003)
    sd = S.synth_state_dict(p, "q8_0", seed=2, max_seq_len=32, trivial_affine=False, weight_std=0.08)
    prompt = S.synth_prompts(3, 4, p.vocab_size, seed=1)
    runs = []
    for seed in (5, 5, 6):
        m = GPT2(rt, p, sd, max_seq_len=32, batch=3)
        runs.append(gpt2_generate(m, prompt, max_length=8, temperature=1.0, top_k=4, seed=seed))
        # the last drawn id is one of the four most likely under the last logits
        top4 = np.argsort(-m.logits(), 1)[:, :4]
        assert all(runs[-1][b, -1] in top4[b] for b in range(3))
        m.close()
    np.testing.assert_array_equal(runs[0], runs[1])
    assert not np.array_equal(runs[0], runs[2])
