"""Host-side pieces of the self-play driver, on CPU: its win rule against the results the
reference's GomokuState reported (golden fixture), and the visit-count -> policy rule."""
import os

import numpy as np

from omoknuni_small_b200 import selfplay

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_result_rule_matches_reference_golden():
    g = np.load(os.path.join(GOLD, "result_golden.npz"))
    ptr, mv = g["row_ptr"], g["moves"]
    got = [selfplay.gomoku_result(mv[ptr[i]:ptr[i + 1]].tolist()) for i in range(len(ptr) - 1)]
    assert np.array_equal(np.asarray(got, np.int8), g["result"])


def test_visits_to_policy():
    # getActionProbabilities: (n / n_max)^(1/T) normalised; T < 0.01 -> one-hot argmax
    assert np.allclose(selfplay.visits_to_policy([0, 3, 1, 0], 1.0), [0, .75, .25, 0])
    assert np.allclose(selfplay.visits_to_policy([0, 3, 1, 0], 0.0), [0, 1, 0, 0])
    p = selfplay.visits_to_policy([4, 2, 0, 2], 0.5)
    assert np.allclose(p, np.array([1, .25, 0, .25]) / 1.5)
    assert not selfplay.visits_to_policy([0, 0], 1.0).any()
