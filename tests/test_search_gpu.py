"""The leaf-parallel search loop on the device.

Against the reference itself a whole search cannot be compared bit for bit (the reference
shuffles children and races on virtual loss).  Two kinds of checks instead:
  * against the CPU restatement (oracle.search_move: descent, expansion, root noise, transposition
    redirect, backup, each citing the reference code it follows) fed the very network outputs the
    device search saw: every array of the tree must be equal bit for bit;
  * invariants, like the reference's own engine tests (tests/mcts/mcts_engine_test.cpp:143-157):
    visit conservation, legality, virtual loss back to zero, consistent expansion, probabilities
    that sum to one, and game-result handling on a forced win."""
import numpy as np
import pytest

from omoknuni_small_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def net(lib):
    from omoknuni_small_b200 import capi
    shapes = synth.net_tensor_shapes(15, 17, 64, 2, 225, 2, 1)
    w = synth.make_weights(shapes, seed=9, init="torch_default", bn="random")
    return capi.Net(17, 15, 2, 64, 225, 2, 1, 256, 256).load(w)


def legal_of(mask_row, n=225):
    return np.unpackbits(mask_row.view(np.uint8), bitorder="little")[:n].astype(bool)


def test_search_invariants(net):
    from omoknuni_small_b200 import capi
    T, sims = 16, 96
    games, _, _, _ = synth.make_gomoku_games(T, 15, seed=5, max_moves=20)
    s = capi.Search(net, n_trees=T, sims_per_move=sims, leaf_batch=128, max_depth=32, c_puct=1.5, virtual_loss=3,
                    dirichlet_epsilon=0.25, seed=1)
    pi, visits, st = s.run(games, temperature=1.0)
    assert st["simulations"] == T * sims and st["evaluations"] == T * sims + T
    assert capi.device_error_code() == 0
    tr = s.tree()
    n = tr["nodes"]
    assert T < n <= T * (sims + 1) and st["nodes"] == n
    assert not tr["VL"].any(), "virtual loss must be back to zero after the backups"
    for t in range(T):
        occupied = np.zeros(225, bool)
        occupied[games[t]] = True
        assert np.array_equal(legal_of(tr["legal_bits"][t]), ~occupied)          # root children = empty cells
        assert visits[t].sum() == sims and tr["node_visits"][t] == sims          # every simulation passes the root once
        assert not visits[t][occupied].any()
        assert abs(pi[t].sum() - 1) < 1e-5 and not pi[t][occupied].any()
        assert np.array_equal(visits[t], tr["N"][t, :225])
    # structure: a child's existence mask is its parent's minus the move, its visits are its edge's
    child = tr["child_node"][:, :225]
    assert child.max() < n and (child >= -1).all()
    parents, slots = np.nonzero(child >= 0)
    for p, a in zip(parents[:400], slots[:400]):
        c = child[p, a]
        lp, lc = legal_of(tr["legal_bits"][p]), legal_of(tr["legal_bits"][c])
        assert lp[a] and not lc[a] and np.array_equal(np.delete(lp, a), np.delete(lc, a))
        assert tr["node_visits"][c] == tr["N"][p, a]
        assert tr["N"][c, :225].sum() <= tr["N"][p, a] - 1                       # the visit(s) that created it stop at the edge
        assert not tr["P"][c, :225][~lc].any() and (tr["P"][c, :225] >= 0).all() and (tr["P"][c, :225] <= 1).all()
    assert len(np.unique(child[child >= 0])) == (child >= 0).sum() == n - T       # one edge per non-root node
    # a second move on the same handle starts from fresh trees
    pi2, visits2, st2 = s.run(games, temperature=0.0)
    assert (visits2.sum(1) == sims).all() and ((pi2 == 1).sum(1) == 1).all() and (pi2.sum(1) == 1).all()
    assert np.array_equal(pi2.argmax(1), visits2.argmax(1))


def open_four(extra_white=0):
    black = [7 * 15 + c for c in (3, 4, 5, 6)]
    white = [0, 14, 210, 224]
    return [m for pair in zip(black, white) for m in pair]


SEARCH_CASES = [
    # name, games (None = seeded openings), trees, simulations per tree and round, rounds, table, noise weight, sign
    ("openings", None, 8, 8, 12, False, 0.25, 1),
    ("openings_table", None, 8, 8, 12, True, 0.25, 1),
    ("long_table", None, 4, 16, 48, True, 0.0, 1),            # 768 simulations per tree: transpositions do occur
    ("open_four_negamax", "four", 4, 16, 12, True, 0.25, -1),  # finished games among the leaves, duplicates in a batch
    ("one_tree", None, 1, 32, 6, True, 0.25, 1),
    # MCTSNode::expand's limits: progressive widening (c, k) -> max(8, c) children per node; the cap on children
    ("widened", None, 8, 8, 12, True, 0.25, 1, {"pw": (2.0, 0.5)}),
    ("widened_20", None, 4, 16, 12, False, 0.25, 1, {"pw": (20.5, 0.5)}),
    ("capped_40", None, 4, 16, 12, True, 0.25, 1, {"max_children": 40}),
    ("capped_and_widened", "four", 4, 16, 12, True, 0.0, -1, {"max_children": 60, "pw": (12.0, 1.0)}),
    # Omok: BLACK's forbidden moves are no children, at the roots and below
    ("omok", "omok", 16, 8, 12, True, 0.25, 1, {"rules": 1}),
    ("omok_widened", "omok", 8, 16, 8, False, 0.25, 1, {"rules": 1, "pw": (16.0, 0.5)}),
    # Renju: overlines, double fours and double threes are no children of BLACK's nodes; BLACK wins with exactly five
    ("renju", "renju", 16, 8, 12, True, 0.25, 1, {"rules": 2}),
    ("renju_negamax", "renju", 8, 16, 8, False, 0.0, -1, {"rules": 2}),
]
SEARCH_CASES = [c if len(c) == 9 else c + ({},) for c in SEARCH_CASES]


@pytest.mark.parametrize("name,games,T,spt,R,table,eps,sign,limits", SEARCH_CASES, ids=[c[0] for c in SEARCH_CASES])
def test_search_equals_the_oracle_on_the_same_network_outputs(net, oracle, name, games, T, spt, R, table, eps, sign, limits):
    """The device search and the CPU restatement, given the same root policies, root noise and per-round
    policy / value arrays: node count, existence masks, child links, visit counts, virtual loss, priors and
    value sums must all be identical.  (Network values are rounded to multiples of 1/256 on both sides so
    that the value sums do not depend on the order of the device's atomic additions.)"""
    from omoknuni_small_b200 import capi
    if games == "four":
        games = [open_four()] * T
    elif games in ("omok", "renju"):
        from test_oracle import load_omok_golden
        all_games, all_legal = load_omok_golden(games + "_golden.npz")
        black_to_move = [k for k, g in enumerate(all_games) if len(g) % 2 == 0]
        pick = (black_to_move + [k for k in range(len(all_games)) if k not in black_to_move])[:T]
        games, root_legal = [all_games[k] for k in pick], all_legal[pick]
    else:
        games, _, _, _ = synth.make_gomoku_games(T, 15, seed=40 + T, max_moves=20)
    s = capi.Search(net, n_trees=T, sims_per_move=spt * R, leaf_batch=T * spt, max_depth=32, c_puct=1.5, virtual_loss=3,
                    dirichlet_alpha=0.3, dirichlet_epsilon=eps, value_sign=sign, transposition_table=table, seed=7,
                    max_children=limits.get("max_children", 0), progressive_widening=limits.get("pw"),
                    rules=limits.get("rules", 0))
    s.debug_hooks(value_quantum=256.0, record_rounds=R)
    target = oracle.widen_target(*limits["pw"]) if "pw" in limits else 0
    for move in range(2):                                          # a second move on the same handle starts clean
        widen = (limits.get("max_children", 1000), target, capi.widening_seed(7, move), limits.get("rules", 0)) if limits else None
        pi, visits, st = s.run(games, temperature=1.0)
        assert capi.device_error_code() == 0
        pol, val, noise = s.record()
        dev = s.tree()
        max_nodes = T * (1 + R * spt)
        ref = oracle.search_move(games, pol[0, :T], noise if eps > 0 else None, eps, pol[1:], val[1:], spt, max_nodes,
                                 c_puct=1.5, vl_value=3, max_depth=32, value_sign=float(sign), value_quantum=256.0,
                                 tt_seed=7 if table else None, widen=widen)
        n = ref["nodes"]
        assert dev["nodes"] == n == st["nodes"], (dev["nodes"], n)
        if limits.get("rules"):
            # the roots' children are the legal moves of the reference's GomokuState(use_omok / use_renju), or a subset
            for t in range(T):
                kids = legal_of(dev["legal_bits"][t])
                assert not (kids & ~root_legal[t]).any() and (target or np.array_equal(kids, root_legal[t]))
            assert any((~root_legal[t] & ~np.isin(np.arange(225), games[t])).any() for t in range(T)), "no forbidden cell among the roots"
        elif limits:
            kids = np.array([legal_of(dev["legal_bits"][k]).sum() for k in range(n)])
            most = min(limits.get("max_children", 1000), target or 1000)
            assert kids.max() == most and (kids[:T] == most).all()
        if limits and eps > 0:                                    # the root noise is a distribution over the root's children
            for t in range(T):
                assert not noise[t, :225][~legal_of(dev["legal_bits"][t])].any() and abs(noise[t].sum() - 1) < 1e-5
        assert st["terminal_leaves"] == ref["terminal_leaves"]
        for key in ("legal_bits", "child_node", "N", "VL", "node_visits"):
            assert np.array_equal(dev[key][:n], ref[key][:n]), key
        assert np.array_equal(dev["P"][:n].view(np.uint32), ref["P"][:n].view(np.uint32)), "priors differ"
        assert np.array_equal(dev["W"][:n].view(np.uint32), ref["W"][:n].view(np.uint32)), "value sums differ"
        assert np.array_equal(visits, ref["N"][:T, :225])
    if name == "long_table":
        child = dev["child_node"][:n, :225]
        assert (child >= 0).sum() > n - T, "the case is meant to contain transpositions"
    if name == "open_four_negamax":
        assert st["terminal_leaves"] > 0


def test_expanded_priors_are_the_clamped_policy_and_root_noise_is_mixed_in(net, oracle):
    """MCTSNode::setPriorProbabilities / addDirichletNoise, stated directly: a node created from leaf i has
    P = clamp(policy[i], 0, 1) on its existing slots and 0 elsewhere; the root has
    (1 - eps) * clamp(policy) + eps * noise with the noise summing to one over the empty cells."""
    from omoknuni_small_b200 import capi
    T, eps = 8, 0.25
    games, _, _, _ = synth.make_gomoku_games(T, 15, seed=3, max_moves=20)
    s = capi.Search(net, n_trees=T, sims_per_move=1, leaf_batch=T, max_depth=8, dirichlet_epsilon=eps, seed=11)
    s.debug_hooks(0.0, 1)
    s.run(games)
    pol, val, noise = s.record()
    tr = s.tree()
    assert tr["nodes"] == 2 * T                                   # one simulation per tree: one new node each
    for t in range(T):
        legal = legal_of(tr["legal_bits"][t])
        assert abs(noise[t, :225][legal].sum() - 1) < 1e-5 and not noise[t, :225][~legal].any() and (noise[t] >= 0).all()
        want = (np.float32(1) - np.float32(eps)) * np.clip(pol[0, t], 0, 1) + np.float32(eps) * noise[t, :225]
        assert np.array_equal(tr["P"][t, :225][legal], want.astype(np.float32)[legal]) and not tr["P"][t, :225][~legal].any()
        a = int(np.nonzero(tr["child_node"][t, :225] >= 0)[0][0])  # the edge the simulation took
        c = tr["child_node"][t, a]
        lc = legal_of(tr["legal_bits"][c])
        assert np.array_equal(tr["P"][c, :225][lc], np.clip(pol[1, t], 0, 1)[lc]) and not tr["P"][c, :225][~lc].any()
    g = np.random.default_rng(0).gamma(0.3, 1.0, 200).astype(np.float32)
    n = oracle.dirichlet_normalize(g)
    assert abs(n.sum() - 1) < 1e-5 and np.array_equal(oracle.dirichlet_normalize(np.zeros(5, np.float32)), np.full(5, 0.2, np.float32))


def test_search_takes_the_win_and_counts_terminals(net):
    """BLACK to move with an open four: the completing move ends the game.  With negamax signs the
    result (+1 for the mover) must pull the visits onto the winning cells.  (Priors are flat, so
    every child is tried once before the win is found; a winning edge carries virtual loss while a
    round is in flight, so it takes about one visit per round after that.)"""
    from omoknuni_small_b200 import capi
    # black: (7,3) (7,4) (7,5) (7,6); white scattered; black to move -> (7,2) or (7,7) wins
    black = [7 * 15 + c for c in (3, 4, 5, 6)]
    white = [0, 14, 210, 224]
    moves = [m for pair in zip(black, white) for m in pair]
    T = 4
    s = capi.Search(net, n_trees=T, sims_per_move=768, leaf_batch=64, max_depth=16, c_puct=1.5, virtual_loss=3,
                    dirichlet_epsilon=0.0, value_sign=-1, seed=3)
    pi, visits, st = s.run([moves] * T, temperature=0.0)
    wins = {7 * 15 + 2, 7 * 15 + 7}
    assert st["terminal_leaves"] > 0
    for t in range(T):
        assert int(visits[t].argmax()) in wins, visits[t].argmax()
        assert min(visits[t][w] for w in wins) >= 20
        others = np.delete(visits[t], list(wins))
        assert others.max() < min(visits[t][w] for w in wins)
    tr = s.tree()
    for t in range(T):                                   # a finished game is never expanded
        for w in wins:
            assert tr["child_node"][t, w] == -1
            if tr["N"][t, w]:
                assert tr["W"][t, w] == tr["N"][t, w]    # every visit backed up the game result +1


def test_terminal_edges_match_the_oracle_rule(net, oracle):
    """After every root child has been tried, the root edges the device treated as finished
    games (never expanded) must be exactly the moves the oracle's rule — pinned to the
    reference's GomokuState on the CPU — calls a win, for roots with threats in all four
    directions, at the board edge, and an overline."""
    from omoknuni_small_b200 import capi

    def interleave(black, white):
        return [m for pair in zip(black, white) for m in pair]
    far = [200, 217, 204, 221, 208, 223]
    roots = [
        interleave([7 * 15 + c for c in (3, 4, 5, 6)], far[:4]),                 # horizontal open four (BLACK to move)
        interleave([r * 15 + 2 for r in (1, 2, 3, 4)], far[:4]),                 # vertical
        interleave([0, 16, 32, 48], [1, 2, 3, 4]),                               # diagonal from the corner
        interleave([14, 28, 42, 56], [1, 2, 3, 5]),                              # anti-diagonal from the corner
        interleave([0, 1, 2, 4, 5], far[:5]),                                    # gap: filling it makes six
        interleave(far[:5], [7 * 15 + c for c in (8, 9, 10, 11)] + [100])[:-1],  # WHITE to move with four
        interleave([10, 11, 12, 13], far[:4]),                                   # four ending at the right edge
        [112],                                                                   # no threat at all
    ]
    T = len(roots)
    # a huge exploration constant makes the search try every root child before it settles
    s = capi.Search(net, n_trees=T, sims_per_move=640, leaf_batch=16 * T, max_depth=8, c_puct=200.0, virtual_loss=3,
                    dirichlet_epsilon=0.0, value_sign=-1, seed=0)
    _, visits, st = s.run(roots, temperature=1.0)
    tr = s.tree()
    for t, root in enumerate(roots):
        occ = set(root)
        want = {a for a in range(225) if a not in occ and oracle.gomoku_result(list(root) + [a]) != 0}
        tried = {a for a in range(225) if tr["N"][t, a] > 0}
        assert tried == set(range(225)) - occ, "every legal root move is tried with this exploration constant"
        got = {a for a in tried if tr["child_node"][t, a] < 0}
        assert got == want, (t, sorted(got), sorted(want))
        for a in want:
            assert tr["W"][t, a] == tr["N"][t, a]                # each visit backed up the result


def test_transposition_table_shares_nodes(net):
    """With the table on, a position reached by two move orders is one node: fewer nodes for the
    same simulations, edges outnumber nodes, and every edge still leads to the position it names."""
    from omoknuni_small_b200 import capi
    T, sims = 8, 640
    games, _, _, _ = synth.make_gomoku_games(T, 15, seed=12, max_moves=10)
    out = {}
    for tt in (False, True):
        s = capi.Search(net, n_trees=T, sims_per_move=sims, leaf_batch=64, max_depth=32, c_puct=1.5, virtual_loss=3,
                        dirichlet_epsilon=0.0, transposition_table=tt, seed=4)
        _, visits, st = s.run(games)
        tr = s.tree()
        assert (visits.sum(1) == sims).all() and not tr["VL"].any()
        out[tt] = (st["nodes"], tr)
    n_off, _ = out[False]
    n_on, tr = out[True]
    assert n_on < n_off, (n_on, n_off)
    child = tr["child_node"][:, :225]
    parents, slots = np.nonzero(child >= 0)
    assert len(parents) > n_on - T                                  # some node has more than one parent edge
    incoming = np.zeros(n_on, np.int64)
    for p, a in zip(parents, slots):
        c = child[p, a]
        lp, lc = legal_of(tr["legal_bits"][p]), legal_of(tr["legal_bits"][c])
        assert lp[a] and not lc[a] and np.array_equal(np.delete(lp, a), np.delete(lc, a))   # same stones either way
        incoming[c] += tr["N"][p, a]
    assert np.array_equal(incoming[T:], tr["node_visits"][T:])      # a shared node counts the visits of all its parents
    # games keep their own trees: a node is reachable from one root only
    owner = np.full(n_on, -1)
    owner[:T] = np.arange(T)
    frontier = list(range(T))
    while frontier:
        p = frontier.pop()
        for c in child[p][child[p] >= 0]:
            assert owner[c] in (-1, owner[p])
            if owner[c] < 0:
                owner[c] = owner[p]
                frontier.append(c)


def test_self_play_records(net, tmp_path, oracle):
    """Games advance together to the end; every record has the reference's fields, legal moves,
    one policy per move, and the result the oracle's rule gives for its move list."""
    import json
    from omoknuni_small_b200 import capi, selfplay
    s = capi.Search(net, n_trees=8, sims_per_move=32, leaf_batch=64, max_depth=16, dirichlet_epsilon=0.25, seed=2)
    sp = selfplay.SelfPlay(s, temperature_threshold=4, max_moves=24, seed=5, out_dir=str(tmp_path))
    recs = sp.generate_games(10)
    assert len(recs) == 10 and len(list(tmp_path.glob("game_*.json"))) >= 10
    for rec in recs:
        assert set(rec) >= {"game_type", "board_size", "winner", "total_time_ms", "game_id", "moves", "policies"}
        mv = rec["moves"]
        assert len(mv) == len(rec["policies"]) <= 24 and len(set(mv)) == len(mv)
        assert all(len(p) == 225 and abs(sum(p) - 1) < 1e-4 for p in rec["policies"])
        assert all(rec["policies"][i][mv[i]] > 0 for i in range(len(mv)))
        res = oracle.gomoku_result(mv)
        assert rec["winner"] == (res if res in (1, 2) else 0)
        assert all(oracle.gomoku_result(mv[:k]) == 0 for k in range(1, len(mv)))     # no move after the end
        assert json.load(open(tmp_path / f"game_{rec['game_id']}.json"))["moves"] == mv
    for mv in ([112], [0, 1, 2, 3, 4, 5, 6, 7, 8], list(range(0, 18))):
        assert selfplay.gomoku_result(mv) == oracle.gomoku_result(mv)


def test_search_argument_errors(net):
    from omoknuni_small_b200 import capi
    with pytest.raises(capi.Error):
        capi.Search(net, n_trees=3, leaf_batch=64)                   # leaf_batch not a multiple of n_trees
    with pytest.raises(capi.Error):
        capi.Search(net, n_trees=64, leaf_batch=1024)                # beyond the network's max_batch (256)
    with pytest.raises(capi.Error):
        capi.Search(net, n_trees=2, leaf_batch=8, rules=3)           # no such rule set
    s = capi.Search(net, n_trees=2, sims_per_move=8, leaf_batch=8)
    with pytest.raises(capi.Error):
        s.run([[5, 5], [1]])                                         # a cell played twice
