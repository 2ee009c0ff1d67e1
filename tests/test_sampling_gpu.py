"""Repetition penalty and the top-k / min-p / top-p cuts on the device, against the plain sampler."""
import numpy as np
import pytest
import torch

from plain.qwen2_plain import penalize_plain, sample_cuts_plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from aegean_tge_b200 import ops as module
    module.core()
    return module


def test_penalty_touches_each_distinct_recent_token_once(ops):
    gen = torch.Generator().manual_seed(1)
    logits = torch.randn(3, 500, generator=gen)
    histories = [[7, 9, 7, 7, 300, 9], list(range(100, 200)) + [7], [4]]
    windows, penalties = [4, 64, 0], [1.3, 2.0, 1.0]
    flat, starts = [], [0]
    for h, w, p in zip(histories, windows, penalties):
        if p != 1.0:
            flat += h[-w:] if w > 0 else h
        starts.append(len(flat))
    out = ops.apply_penalty(logits.to(DEV), torch.tensor(flat, dtype=torch.int32, device=DEV),
                            torch.tensor(starts, dtype=torch.int32, device=DEV),
                            torch.tensor(penalties, device=DEV)).cpu().numpy()
    for r in range(3):
        expected = penalize_plain(logits[r].numpy(), histories[r], penalties[r], windows[r])
        assert np.array_equal(out[r], expected), r
    assert not np.array_equal(out[0], logits[0].numpy()) and np.array_equal(out[2], logits[2].numpy())


@pytest.mark.parametrize("vocab", [331, 5000])
@pytest.mark.parametrize("top_k,top_p,min_p", [(5, 1.0, 0.0), (0, 0.7, 0.0), (0, 1.0, 0.05), (40, 0.9, 0.02), (1, 1.0, 0.0),
                                               (0, 0.999, 0.0)])
def test_cuts_pick_what_the_plain_sampler_picks(ops, vocab, top_k, top_p, min_p):
    gen = torch.Generator().manual_seed(vocab + top_k)
    rows = 8
    logits = torch.randn(rows, vocab, generator=gen) * 3.0
    temps = [0.7, 1.0, 1.5, 0.3, 0.7, 1.0, 2.0, 0.9]
    uniforms = [0.03, 0.5, 0.97, 0.25, 0.61, 0.999, 0.42, 0.0]
    mk = lambda v, dt: torch.tensor(v, dtype=dt, device=DEV)
    ids = ops.sample_cuts(logits.to(DEV), mk(temps, torch.float32), mk([top_k] * rows, torch.int32),
                          mk([top_p] * rows, torch.float32), mk([min_p] * rows, torch.float32),
                          mk(uniforms, torch.float32)).cpu().tolist()
    for r in range(rows):
        expected = sample_cuts_plain(logits[r].numpy(), temps[r], top_k, top_p, min_p, uniforms[r])
        if ids[r] != expected:
            # The device forms its sums in another order than the sequential float32 walk.  A float32 sum of n
            # terms is exact to about n * 2^-24 of the total, so the two picks may differ only when the
            # probability mass lying between them in the sorted order is within that rounding.
            z = logits[r].double()
            prob = torch.exp((z - z.max()) / temps[r])
            order = sorted(range(vocab), key=lambda i: (-float(prob[i]), i))
            a, b = sorted((order.index(ids[r]), order.index(expected)))
            between = float(sum(prob[i] for i in order[a:b])) / float(prob.sum())
            assert between < vocab * 2.0 ** -23, (r, ids[r], expected, between)


@pytest.mark.parametrize("spread,top_k,top_p,min_p", [(4.0, 0, 0.9, 0.0), (4.0, 50, 0.95, 0.0), (4.0, 0, 1.0, 0.001),
                                                     (0.3, 0, 0.9, 0.0), (0.3, 6000, 0.5, 0.0), (0.0, 0, 0.5, 0.0)])
def test_cuts_at_a_real_vocabulary(ops, spread, top_k, top_p, min_p):
    """152,064 scores per row.  Peaked rows (a spread of 4) are settled among a few thousand candidates sorted in
    shared memory; flat rows (0.3: the nucleus is most of the vocabulary; 0: all scores equal, every probability
    ties and the lower index goes first) and a top-k beyond the candidates take the full sort.  Both give the
    plain sampler's token, up to the rounding of the sums."""
    vocab, rows = 152064, 3
    gen = torch.Generator().manual_seed(int(spread * 10) + top_k)
    logits = torch.randn(rows, vocab, generator=gen) * spread
    temps, uniforms = [0.8, 1.0, 1.3], [0.37, 0.93, 0.05]
    mk = lambda v, dt: torch.tensor(v, dtype=dt, device=DEV)
    args = (mk(temps, torch.float32), mk([top_k] * rows, torch.int32), mk([top_p] * rows, torch.float32),
            mk([min_p] * rows, torch.float32), mk(uniforms, torch.float32))
    ids = ops.sample_cuts(logits.to(DEV), *args).cpu().tolist()
    assert ids == ops.sample_cuts(logits.to(DEV), *args).cpu().tolist()          # the same token every time
    for r in range(rows):
        z = logits[r].double()
        prob = torch.exp((z - z.max()) / temps[r])
        order = torch.tensor(sorted(range(vocab), key=lambda i: (-float(prob[i]), i)))
        # the plain walk in float64 over the sorted order (the float32 walk is the same up to the rounding let through below)
        keep = min(top_k, vocab) if top_k > 0 else vocab
        kept = order[:keep]
        if min_p > 0.0:
            kept = kept[prob[kept] >= min_p * prob[kept[0]]]
        mass = torch.cumsum(prob[kept], 0)
        limit = len(kept)
        if top_p < 1.0:
            limit = int(torch.searchsorted(mass / mass[-1], torch.tensor(top_p, dtype=torch.float64))) + 1
        target = uniforms[r] * float(mass[limit - 1])
        expected_position = min(int(torch.searchsorted(mass[:limit], torch.tensor(target, dtype=torch.float64))), limit - 1)
        position = int((kept == ids[r]).nonzero()[0]) if ids[r] in kept.tolist() else -1
        assert position >= 0, (r, ids[r])
        a, b = sorted((position, expected_position))
        between = float(prob[kept[a:b]].sum()) / float(mass[-1])
        assert between < vocab * 2.0 ** -23, (r, position, expected_position, between)


def test_cuts_do_not_depend_on_the_batch(ops):
    """A row of a large vocabulary is shared by eight blocks when it is sampled alone and by fewer, down to one,
    in a large batch.  Its token must be the same: the total that top-p refers to is added as integers and the
    sorted candidates in chunks of a fixed size, so neither depends on who scanned what.  Many draws near every
    kind of edge (a nucleus that ends between two near-equal candidates, a top-k, a floor) in three batch sizes."""
    vocab = 152064
    gen = torch.Generator().manual_seed(77)
    kinds = [(0, 0.9, 0.0), (40, 0.95, 0.0), (0, 1.0, 0.002), (0, 0.5, 0.0), (3000, 0.8, 0.0), (0, 0.97, 1e-4)]
    rows = 24
    logits = (torch.randn(rows, vocab, generator=gen) * torch.linspace(1.5, 5.0, rows)[:, None]).to(DEV)
    temps = torch.linspace(0.6, 1.4, rows)
    uniforms = torch.rand(rows, generator=gen)
    top_k = torch.tensor([kinds[r % len(kinds)][0] for r in range(rows)], dtype=torch.int32)
    top_p = torch.tensor([kinds[r % len(kinds)][1] for r in range(rows)])
    min_p = torch.tensor([kinds[r % len(kinds)][2] for r in range(rows)])

    def run(pick):
        take = lambda t: t[pick].to(DEV).contiguous()
        return ops.sample_cuts(logits[pick.to(DEV)].contiguous(), take(temps), take(top_k), take(top_p), take(min_p),
                               take(uniforms)).cpu().tolist()

    alone = [run(torch.tensor([r]))[0] for r in range(rows)]                    # eight blocks per row
    together = run(torch.arange(rows))                                          # 24 rows: four blocks per row
    many = run(torch.arange(rows).repeat(5))                                    # 120 rows: one block per row
    assert together == alone
    assert many == alone * 5


def test_cut_draws_stay_inside_the_cut_and_follow_the_distribution(ops):
    """Many draws with top-k 3 from a known distribution: nothing outside the top three, shares as renormalised."""
    from aegean_tge_b200.sampling import XorShift32
    probs = torch.tensor([0.4, 0.05, 0.3, 0.05, 0.2])
    n = 3000
    logits = torch.log(probs)[None, :].repeat(n, 1)
    rng = XorShift32(5)
    uniforms = torch.tensor([rng.next_uniform() for _ in range(n)])
    mk = lambda v, dt: torch.full((n,), v, dtype=dt, device=DEV)
    ids = ops.sample_cuts(logits.to(DEV), mk(1.0, torch.float32), mk(3, torch.int32), mk(1.0, torch.float32),
                          mk(0.0, torch.float32), uniforms.to(DEV)).cpu()
    counts = torch.bincount(ids.long(), minlength=5).double()
    assert counts[1] == 0 and counts[3] == 0
    expected = torch.tensor([0.4, 0.0, 0.3, 0.0, 0.2]).double() / 0.9 * n
    keep = expected > 0
    chi2 = float((((counts - expected) ** 2)[keep] / expected[keep]).sum())
    assert chi2 < 15.2                  # 2 degrees of freedom, p ~ 5e-4


def test_engine_samples_with_cuts_and_penalty(model_dirs):
    """Through the entry point: cuts and penalty per request, reproducible for a seed, penalty changes greedy output."""
    from aegean_tge_b200 import Engine, SamplingParams
    engine = Engine(model_dirs["B"], dtype="float32", context=128, max_tokens=512, max_requests=4)
    prompt = [3, 14, 15, 92, 65]
    cut = SamplingParams(temperature=0.9, top_k=20, top_p=0.9, min_p=0.01, repeat_penalty=1.2, seed=9)
    a = engine.generate(prompt, n=12, sampling=cut)
    b = engine.generate(prompt, n=12, sampling=cut)
    assert a == b and len(a) == 12
    plain_greedy = engine.generate(prompt, n=12)
    penalised = engine.generate(prompt, n=12, sampling=SamplingParams(repeat_penalty=50.0, penalty_window=0))
    assert len(set(penalised)) == len(penalised)            # a huge penalty never repeats a token
    assert penalised[0] == plain_greedy[0] or plain_greedy[0] in prompt
    mixed = engine.generate([prompt, prompt], n=6, sampling=[cut, SamplingParams()])
    assert mixed[0] == a[:6] and mixed[1] == plain_greedy[:6]
