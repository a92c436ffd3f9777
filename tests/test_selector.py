"""The block drafter's low-rank selector: the walk against a brute-force restatement, keyed walks, refusals, and the lattice form."""
import numpy as np
import pytest

from rexl3_b200.sampling import Sampling, choose
from rexl3_b200.spec import Policy, SelectorError, SelectorInputs, best_first, selector_lattice, selector_walk


def make(seed=0, T=5, k=4, rank=6, vocab=50):
    rng = np.random.default_rng(seed)
    pred = rng.normal(size=(vocab, rank)).astype(np.float32)
    succ = rng.normal(size=(vocab, rank)).astype(np.float32)
    cands = [rng.choice(vocab, size=k, replace=False).tolist() for _ in range(T)]
    unary = [rng.normal(size=k).astype(np.float32).tolist() for _ in range(T)]
    hidden = [rng.normal(size=rank).astype(np.float32) for _ in range(T)]
    return SelectorInputs(cands, unary, hidden, lambda t: pred[t], lambda t: succ[t]), pred, succ


def test_greedy_walk_is_the_argmax_of_unary_plus_coupling():
    for seed in range(5):
        x, pred, succ = make(seed)
        path = selector_walk(7, x)
        prev = 7
        for p, tok in enumerate(path):
            sc = [u + float(np.sum(pred[prev] * x.hidden[p] * succ[c])) for c, u in zip(x.candidates[p], x.unary[p])]
            best = max(range(len(sc)), key=lambda i: (sc[i], -x.candidates[p][i]))
            assert tok == x.candidates[p][best]
            prev = tok
        # the coupling matters: with a zero hidden state the walk is the per-position unary argmax
        x0 = SelectorInputs(x.candidates, x.unary, [np.zeros(6, np.float32)] * 5, x.predecessor, x.successor)
        assert selector_walk(7, x0) == [c[int(np.argmax(u))] for c, u in zip(x.candidates, x.unary)]
    assert any(selector_walk(7, make(s)[0]) != [c[int(np.argmax(u))] for c, u in zip(make(s)[0].candidates, make(s)[0].unary)] for s in range(5))


def test_keyed_walk_draws_with_the_targets_noise_at_each_position():
    x, pred, succ = make(3)
    s = Sampling(seed=99, temperature=0.9, top_k=2, top_p=0.9)
    path = selector_walk(7, x, s, first_position=100)
    prev = 7
    for p, tok in enumerate(path):
        sc = [float(np.float32(u + np.sum(pred[prev] * x.hidden[p] * succ[c]))) for c, u in zip(x.candidates[p], x.unary[p])]
        want = choose(sc, x.candidates[p], 100 + p, Sampling(seed=99, temperature=0.9, top_k=len(sc), top_p=0.9))
        assert tok == want or abs(max(sc) - sorted(sc)[-2]) < 1e-5
        prev = tok
    assert selector_walk(7, x, s, first_position=100) == path
    assert any(selector_walk(7, x, s, first_position=q) != path for q in range(101, 140))


def test_refusals_name_the_fault():
    x, _, _ = make(1)
    with pytest.raises(SelectorError, match="5 candidate lists, 4 unary rows"):
        selector_walk(0, SelectorInputs(x.candidates, x.unary[:4], x.hidden, x.predecessor, x.successor))
    bad = [list(u) for u in x.unary]
    bad[2] = bad[2][:3]
    with pytest.raises(SelectorError, match="position 2: 4 candidates but 3 unary"):
        selector_walk(0, SelectorInputs(x.candidates, bad, x.hidden, x.predecessor, x.successor))
    with pytest.raises(SelectorError, match="predecessor rank 6 but hidden rank 5"):
        selector_walk(0, SelectorInputs(x.candidates, x.unary, [h[:5] for h in x.hidden], x.predecessor, x.successor))
    nan = [list(u) for u in x.unary]
    nan[1][0] = float("nan")
    e = pytest.raises(SelectorError, selector_walk, 0, SelectorInputs(x.candidates, nan, x.hidden, x.predecessor, x.successor))
    assert e.value.kind == "sampling"
    empty = SelectorInputs([[]] + x.candidates[1:], [[]] + x.unary[1:], x.hidden, x.predecessor, x.successor)
    assert pytest.raises(SelectorError, selector_walk, 0, empty).value.kind == "sampling"


def test_lattice_carries_the_coupling_per_parent_and_the_tree_follows_the_walk():
    x, pred, succ = make(4)
    lat = selector_lattice(7, x)
    assert len(lat.edge) == 5 and len(lat.edge[0]) == 1 and len(lat.edge[1]) == 4 and len(lat.edge[1][0]) == 4
    p, i, j = 3, 2, 1
    want = float(np.sum(pred[x.candidates[p - 1][i]] * x.hidden[p] * succ[x.candidates[p][j]]))
    assert abs(lat.edge[p][i][j] - want) < 1e-4
    # a tree of one child per node under the selector's own scores is the greedy walk
    tree = best_first(lat, 5, Policy(edge=1.0, noise=0.0, scale=1.0, branch=1))
    assert tree.tokens == selector_walk(7, x) and tree.parents == [-1, 0, 1, 2, 3]
    # with four children per node the walk's path is still in the tree's first levels and siblings hang under their own parents
    wide = best_first(lat, 12, Policy(edge=1.0, noise=0.0, scale=1.0, branch=4))
    assert wide.tokens[0] == selector_walk(7, x)[0] and len(wide) == 12
