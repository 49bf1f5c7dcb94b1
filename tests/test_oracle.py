"""Pins the CPU oracle: against the golden fixtures produced by the reference
project's own classes, against the known-answer cases of the reference's unit
tests, and (when oracle/_ref was built) against the reference classes live."""
import hashlib
import os

import numpy as np
import pytest

from omoknuni_small_b200 import synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def sha(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def tiny_tree(N, W, P, VL, n_parent):
    n = len(N)
    pitch, mw = synth.tree_pitch(n), synth.tree_mask_words(n)
    t = {"N": np.zeros((1, pitch), np.int32), "W": np.zeros((1, pitch), np.float32), "P": np.zeros((1, pitch), np.float32),
         "VL": np.zeros((1, pitch), np.int32), "legal_bits": np.zeros((1, mw), np.uint32),
         "node_visits": np.array([n_parent], np.int32), "n_children": n}
    t["N"][0, :n], t["W"][0, :n], t["P"][0, :n], t["VL"][0, :n] = N, W, P, VL
    t["legal_bits"][0, 0] = (1 << n) - 1
    return t


# ---- known answers restated from the reference's unit tests ------------------------
def test_child_selection_known_answers(oracle):
    # tests/mcts/mcts_node_test.cpp:237-268 — priors .7/.2/.1, parent visited once, c = 1.0
    t = tiny_tree([0, 0, 0], [0, 0, 0], [.7, .2, .1], [0, 0, 0], 1)
    assert oracle.puct_select(t, c_puct=1.0)[0] == 0
    # after child0.update(-1) a different child is chosen
    t = tiny_tree([1, 0, 0], [-1, 0, 0], [.7, .2, .1], [0, 0, 0], 1)
    assert oracle.puct_select(t, c_puct=1.0)[0] != 0


def test_virtual_loss_known_answers(oracle):
    # tests/mcts/mcts_node_test.cpp:271-298 — equal priors; VL on the selected child moves the choice, removing restores it
    t = tiny_tree([0, 0, 0], [0, 0, 0], [1 / 3] * 3, [0, 0, 0], 1)
    first = oracle.puct_select(t, c_puct=1.0)[0]
    t["VL"][0, first] += 1
    assert oracle.puct_select(t, c_puct=1.0)[0] != first
    t["VL"][0, first] -= 1
    assert oracle.puct_select(t, c_puct=1.0)[0] == first
    # tests/mcts/virtual_loss_test.cpp:195-224 — five equal children (10 visits, mean .5), parent 50, VL 3 on one, c = 1.5
    t = tiny_tree([10] * 5, [5.0] * 5, [.2] * 5, [3, 0, 0, 0, 0], 50)
    assert oracle.puct_select(t, c_puct=1.5)[0] != 0
    # :160-193 stacking 1,2,3 then remove(3) twice -> 3, 0 ; :282-308 removing more than present clamps to 0
    assert list(oracle.vl_ops(0, [1, 2, 3, -3, -3])) == [1, 3, 6, 3, 0]
    assert list(oracle.vl_ops(0, [2, -5, 0, 0])) == [2, 0, 0, 0]


def test_backprop_known_answer(oracle):
    # tests/mcts/mcts_node_test.cpp:301-313 — two updates 1.0 and 0.5 -> 2 visits, mean 0.75
    t = tiny_tree([0], [0], [1], [0], 0)
    paths = np.zeros((1, 1, 2), np.int32)
    for v in (1.0, 0.5):
        oracle.backup(t, paths, [1], [v], vl_value=0)
    assert t["N"][0, 0] == 2 and t["W"][0, 0] / t["N"][0, 0] == 0.75 and t["node_visits"][0] == 2


# ---- golden fixtures made by the reference's own classes ---------------------------
@pytest.mark.parametrize("tag", ["g225", "c4672", "n3"])
def test_selection_matches_reference_golden(oracle, tag):
    g = np.load(os.path.join(GOLD, "select_golden.npz"))
    n_nodes, nc, seed = g[tag + "_shape"]
    t = synth.make_selection_tree(int(n_nodes), int(nc), seed=int(seed))
    assert sha(t["N"], t["W"], t["P"], t["VL"], t["legal_bits"], t["node_visits"]) == str(g[tag + "_inputs_sha256"])
    rows = np.arange(n_nodes)
    vl0 = t["VL"].copy()
    sel = oracle.puct_select(t, c_puct=1.5, vl_value=3, apply_vl=True)
    assert np.array_equal(sel, g[tag + "_sel"])
    assert np.array_equal(t["VL"][rows, sel], g[tag + "_vl_after_apply"])
    oracle.vl_revert(t, sel, 3)
    assert np.array_equal(t["VL"][rows, sel], g[tag + "_vl_after_revert"])
    assert np.array_equal(t["VL"], vl0)            # apply then revert conserves every counter


def load_encode_golden():
    g = np.load(os.path.join(GOLD, "encode_golden.npz"))
    shape = tuple(g["planes_shape"])
    planes = np.unpackbits(g["planes_bits"])[: int(np.prod(shape))].reshape(shape).astype(np.float32)
    games = [g["moves"][g["row_ptr"][i]:g["row_ptr"][i + 1]].astype(np.int32) for i in range(shape[0])]
    hist = np.full((shape[0], 16), -1, np.int16)
    nh = np.zeros(shape[0], np.uint8)
    for i, mv in enumerate(games):
        h = mv[::-1][:16]
        hist[i, :len(h)] = h
        nh[i] = len(h)
    return games, hist, nh, g["to_move"], planes, bool(g["planes_is_binary"])


def test_encoder_matches_reference_golden(oracle):
    games, hist, nh, tm, planes, binary = load_encode_golden()
    assert binary                                   # the reference's planes are all 0/1, so bf16 is exact
    enc = oracle.gomoku_encode(hist, nh, tm, 15, 19)
    assert np.array_equal(enc, planes)
    assert not planes[:, 17:].any()                 # attack/defense planes of the reference's CPU path are zero
    assert np.array_equal(oracle.gomoku_encode(hist, nh, tm, 15, 17), planes[:, :17])


def load_go_golden(tag):
    """Positions of the reference's GoState and its planes (tests/golden/make_golden.py): stones
    [n,S,S] int8, ko [n] int32, to_move [n] u8, legal [n,S,S] u8, planes [n,10,S,S] fp32."""
    g = np.load(os.path.join(GOLD, "go_golden.npz"))
    stones = g[tag + "_stones"]
    n, S = stones.shape[0], stones.shape[1]
    legal = np.unpackbits(g[tag + "_legal"], axis=1)[:, :S * S].reshape(n, S, S)
    return stones, g[tag + "_ko"], g[tag + "_to_move"], legal, g[tag + "_planes"]


@pytest.mark.parametrize("tag", ["s9", "s19"])
def test_go_encoder_matches_reference_golden(oracle, tag):
    stones, ko, tm, legal, planes = load_go_golden(tag)
    assert (ko >= 0).any() or tag == "s19"            # the 9x9 set holds positions with a ko point
    assert (planes[:, 8] > 0).any() and (planes[:, 9] > 0).any() and (planes[:, 3] > 0).any()
    assert np.array_equal(oracle.go_encode(stones, ko, tm, legal), planes)


def load_chess_golden():
    """Positions of the reference's ChessState and its planes (tests/golden/make_golden.py)."""
    g = np.load(os.path.join(GOLD, "chess_golden.npz"))
    return g["pieces"], g["meta"], g["legal_to"], g["planes"]


def test_chess_encoder_matches_reference_golden(oracle):
    pieces, meta, legal_to, planes = load_chess_golden()
    assert (meta[:, 2] >= 0).any() and len(np.unique(meta[:, 1])) > 4 and set(np.unique(meta[:, 0])) == {1, 2}
    assert np.array_equal(oracle.chess_encode(pieces, meta, legal_to), planes)


def test_game_result_matches_reference_golden(oracle):
    g = np.load(os.path.join(GOLD, "result_golden.npz"))
    ptr, mv = g["row_ptr"], g["moves"]
    got = [oracle.gomoku_result(mv[ptr[i]:ptr[i + 1]]) for i in range(len(ptr) - 1)]
    assert np.array_equal(np.asarray(got, np.int8), g["result"])
    assert (g["result"] != 0).sum() >= 10                        # the fixture does contain finished games


def test_game_result_known_cases(oracle):
    def interleave(black, white):
        return [m for pair in zip(black, white) for m in pair]
    far = [200, 202, 204, 206, 208, 210]
    assert oracle.gomoku_result(interleave([0, 1, 2, 3, 4], far)[:-1]) == 1            # five in a row
    assert oracle.gomoku_result(interleave([0, 1, 2, 4, 5, 3], far)[:-1]) == 1         # six: overline wins in freestyle
    assert oracle.gomoku_result(interleave([0, 16, 32, 48, 64], far)[:-1]) == 1        # diagonal
    assert oracle.gomoku_result(interleave([14, 28, 42, 56, 70], far)[:-1]) == 1       # anti-diagonal
    assert oracle.gomoku_result(interleave([0, 1, 2, 3], far)) == 0                     # four is not enough
    assert oracle.gomoku_result(interleave(far, [0, 15, 30, 45, 60])) == 2             # WHITE, vertical
    assert oracle.gomoku_result([11, 12, 13, 14, 15][:0]) == 0                          # empty game
    assert oracle.gomoku_result(interleave([10, 11, 12, 13, 14 + 15], far)[:-1]) == 0  # no wrap over the board edge


def load_net_golden_a():
    g = np.load(os.path.join(GOLD, "net_golden.npz"))
    cin, S, blocks, F, A, pc, vc = [int(v) for v in g["a_cfg"]]
    shapes = dict(synth.net_tensor_shapes(S, cin, F, blocks, A, pc, vc))
    w = {k[4:]: g[k].astype(np.float32).reshape(shapes[k[4:]]) for k in g.files if k.startswith("a_w_")}
    shape = tuple(g["a_x_shape"])
    x = np.unpackbits(g["a_x_bits"])[: int(np.prod(shape))].reshape(shape).astype(np.float32)
    return dict(cin=cin, S=S, blocks=blocks, F=F, A=A, pc=pc, vc=vc), w, x, g["a_logp"], g["a_value"]


def load_net_golden_b():
    g = np.load(os.path.join(GOLD, "net_golden.npz"))
    shapes = synth.net_tensor_shapes(15, 17, 64, 10, 225, 32, 32)
    w = synth.make_weights(shapes, seed=42, init="torch_default", bn="random")
    x = synth.make_stone_planes(8, 15, 17, seed=1000)
    assert sha(*[w[k] for k, _ in shapes]) == str(g["b_weights_sha256"]) and sha(x) == str(g["b_x_sha256"])
    return w, x, g["b_logp"], g["b_value"]


def test_network_restatement_matches_reference_golden():
    from oracle import net_ref
    cfg, w, x, logp, value = load_net_golden_a()
    logits, v = net_ref.forward(w, x)
    assert np.abs(net_ref.log_softmax(logits) - logp).max() < 2e-6 and np.abs(v - value).max() < 2e-6
    w, x, logp, value = load_net_golden_b()
    logits, v = net_ref.forward(w, x)
    assert np.abs(net_ref.log_softmax(logits) - logp).max() < 2e-5 and np.abs(v - value).max() < 2e-6
    # what the reference's own test asserts (tests/nn/neural_network_test.cpp:38-72)
    assert logits.shape == (8, 225) and np.all(np.abs(v) <= 1) and np.allclose(np.exp(logp).sum(1), 1, atol=1e-5)


# ---- live against the reference classes (only where oracle/_ref exists) -------------
def _need_ref(oracle, which):
    ok = oracle.have_ref_tree() if which == "tree" else oracle.have_ref_net()
    if not ok:
        pytest.skip("oracle/_ref not built here (the reference checkout is absent)")


def test_selection_live_against_mctsnode(oracle):
    _need_ref(oracle, "tree")
    for nc, n_nodes, seed in ((225, 2048, 70), (362, 128, 71), (7, 256, 72)):
        t = synth.make_selection_tree(n_nodes, nc, seed=seed)
        sel_ref, a, r, _ = oracle.ref_select(t, c_puct=1.5, vl_value=3)
        assert np.array_equal(oracle.puct_select(t, c_puct=1.5), sel_ref)
    ops = [1, 2, 3, -3, -3, -5, 0, 0, 4, -1, -10, 0]
    assert np.array_equal(oracle.vl_ops(0, ops), oracle.ref_vl_ops(0, ops))


def test_backup_live_against_mctsnode(oracle):
    _need_ref(oracle, "tree")
    rng = np.random.default_rng(3)
    for _ in range(20):
        d = int(rng.integers(1, 9))
        N = rng.integers(0, 20, d).astype(np.int32)
        W = (N * rng.uniform(-1, 1, d)).astype(np.float32)
        VL = rng.integers(0, 8, d).astype(np.int32)
        leaf = float(np.float32(rng.uniform(-1, 1)))
        # oracle on an edge table: path node i is edge (i, 0)
        t = {"N": np.zeros((d, 4), np.int32), "W": np.zeros((d, 4), np.float32), "VL": np.zeros((d, 4), np.int32),
             "node_visits": np.zeros(d, np.int32)}
        t["N"][:, 0], t["W"][:, 0], t["VL"][:, 0] = N, W, VL
        paths = np.zeros((1, d, 2), np.int32)
        paths[0, :, 0] = np.arange(d)
        oracle.backup(t, paths, [d], [leaf], vl_value=3)
        rN, rVL, rmean = oracle.ref_backup_path(N, W, VL, leaf, 3)
        assert np.array_equal(t["N"][:, 0], rN) and np.array_equal(t["VL"][:, 0], rVL)
        assert np.array_equal((t["W"][:, 0] / t["N"][:, 0]).astype(np.float32), rmean)


def test_encoder_live_against_gomokustate(oracle):
    _need_ref(oracle, "tree")
    games, hist, nh, tm = synth.make_gomoku_games(96, 15, seed=9)
    ref, _ = oracle.ref_gomoku_encode_batch(games, 15)
    assert np.array_equal(oracle.gomoku_encode(hist, nh, tm, 15, 19), ref)
    games, hist, nh, tm = synth.make_gomoku_games(16, 9, seed=10, max_moves=30)
    ref, _ = oracle.ref_gomoku_encode_batch(games, 9)
    assert np.array_equal(oracle.gomoku_encode(hist, nh, tm, 9, 19), ref)


def test_go_encoder_live_against_gostate(oracle):
    """The C restatement against GoState::getEnhancedTensorRepresentation on fresh random games."""
    _need_ref(oracle, "tree")
    gs = oracle.random_go_games(16, 9, seed=4242, max_moves=90) + oracle.random_go_games(2, 13, seed=4243, max_moves=120)
    for g in gs:
        got = oracle.go_encode(g["stones"][None], np.array([g["ko_point"]], np.int32), np.array([g["to_move"]], np.uint8),
                               g["legal"][None])[0]
        assert np.array_equal(got, g["planes"])


def test_chess_encoder_live_against_chessstate(oracle):
    """The C restatement against ChessState::getEnhancedTensorRepresentation on fresh random games."""
    _need_ref(oracle, "tree")
    pieces, meta, legal_to, planes = oracle.ref_chess_positions(60, seed=777, max_plies=200)
    assert np.array_equal(oracle.chess_encode(pieces, meta, legal_to), planes)


def test_gomoku_planes3_live_against_gomokustate(oracle):
    """The 3-plane representation against GomokuState::getTensorRepresentation."""
    _need_ref(oracle, "tree")
    games, _, _, _ = synth.make_gomoku_games(40, 15, seed=31, max_moves=120)
    for g in games[:40]:
        st, tm = oracle.stones_from_moves(g, 15)
        _, p3, tm_ref = oracle.ref_gomoku_planes(g, 15)
        assert tm == tm_ref
        assert np.array_equal(oracle.gomoku_planes3(st[None], np.array([tm], np.uint8))[0], p3)


def test_game_result_live_against_gomokustate(oracle):
    _need_ref(oracle, "tree")
    rng = np.random.default_rng(8)
    games, _, _, _ = synth.make_gomoku_games(60, 15, seed=707, max_moves=150)
    n_done = 0
    for g in games:
        occ = set(int(x) for x in g)
        for a in rng.permutation(225)[:20]:
            if int(a) in occ:
                continue
            mv = [int(x) for x in g] + [int(a)]
            r = oracle.ref_gomoku_result(mv)
            assert r == oracle.gomoku_result(mv)
            n_done += r != 0
    assert n_done > 0
    six = [0, 200, 1, 202, 2, 204, 4, 206, 5, 208, 3]
    assert oracle.ref_gomoku_result(six) == oracle.gomoku_result(six) == 1


def test_network_live_against_resnetmodel(oracle):
    _need_ref(oracle, "net")
    from oracle import net_ref
    net = oracle.RefNet(17, 9, 2, 64, 81, seed=5)       # the shape of tests/nn/neural_network_test.cpp:17 with 64 filters
    shapes = dict(synth.net_tensor_shapes(9, 17, 64, 2, 81, 32, 32))
    w = {k: a.reshape(shapes[k]) for k, a in net.state().items() if "num_batches" not in k}
    x = synth.make_stone_planes(4, 9, 19, seed=1)        # 19 planes in, 17 used (channel adaptation)
    lp, v, _ = net.forward(x)
    logits, val = net_ref.forward(w, x)
    assert np.abs(net_ref.log_softmax(logits) - lp).max() < 2e-6 and np.abs(val - v).max() < 2e-6


def test_search_round_restatement_invariants(oracle):
    """oracle.search_move (descent -> expansion -> backup per round) on seeded policy / value arrays: visits are
    conserved, virtual loss returns to zero, a child's existence mask is its parent's minus the move, priors are
    the clamped policy rows, and with the table on positions reached by two move orders share one node."""
    rng = np.random.default_rng(5)
    T, spt, R = 2, 8, 40
    games = [[112, 113], [0, 224, 16]]
    root_pol = rng.dirichlet(np.full(225, 0.5), T).astype(np.float32)
    # every leaf gets the same policy, peaked on six cells: the trees go deep over permutations of those cells
    row = np.full(225, 0.001, np.float32)
    row[[40, 41, 42, 55, 56, 57]] = 0.16
    pol = np.broadcast_to(row, (R, T * spt, 225)).copy()
    val = (rng.integers(-256, 257, (R, T * spt)) / 256.0).astype(np.float32)
    noise = np.zeros((T, 228), np.float32)
    out = {}
    for tt in (None, 3):
        tr = oracle.search_move(games, root_pol, noise, 0.0, pol, val, spt, T * (1 + R * spt), value_quantum=256.0, tt_seed=tt)
        n = tr["nodes"]
        assert not tr["VL"].any()
        assert (tr["N"][:T, :225].sum(1) == spt * R).all() and (tr["node_visits"][:T] == spt * R).all()
        child = tr["child_node"][:n, :225]
        parents, slots = np.nonzero(child >= 0)
        incoming = np.zeros(n, np.int64)
        for p, a in zip(parents, slots):
            c = child[p, a]
            lp = np.unpackbits(tr["legal_bits"][p].view(np.uint8), bitorder="little")[:225]
            lc = np.unpackbits(tr["legal_bits"][c].view(np.uint8), bitorder="little")[:225]
            assert lp[a] and not lc[a] and np.array_equal(np.delete(lp, a), np.delete(lc, a))
            assert not tr["P"][c, :225][lc == 0].any()
            incoming[c] += tr["N"][p, a]
        assert np.array_equal(incoming[T:], tr["node_visits"][T:n])
        out[tt] = (n, len(parents))
    assert out[None][1] == out[None][0] - T            # a tree: one edge per node
    assert out[3][0] < out[None][0] and out[3][1] > out[3][0] - T   # shared nodes: fewer nodes, more edges than nodes


def test_widening_count_and_choice_against_the_reference_expand(oracle):
    """MCTSNode::expand's limits on a node's children (src/mcts/mcts_node.cpp:283-340).  The count progressive
    widening asks for is pinned to the compiled reference (its random subset itself cannot be: it is seeded from
    the operating system); the restated choice keeps that many of the legal moves, is a function of (seed, node,
    move) only, and takes every move about equally often."""
    assert oracle.widen_target(2.0, 0.5) == 8 and oracle.widen_target(20.5, 0.5) == 20
    assert oracle.widen_target(0.5, 5.0) == 8 and oracle.widen_target(1.0, 10.0, visits=3) == 4 ** 10
    moves = [112, 113, 98]
    empty = np.ones(225, bool)
    empty[moves] = False
    words = np.packbits(np.concatenate([empty, np.zeros(31, bool)]), bitorder="little").view(np.uint32)
    legal_of = lambda w: np.unpackbits(w.view(np.uint8), bitorder="little")[:225].astype(bool)
    if oracle.have_ref_tree():
        for use, c, k in [(True, 2.0, 0.5), (True, 20.5, 0.5), (True, 0.5, 5.0), (True, 300.0, 1.0), (False, 2.0, 0.5)]:
            acts = oracle.ref_expand_gomoku(moves, use, c, k)
            want = min(222, oracle.widen_target(c, k)) if use else 222
            assert len(acts) == want == len(set(acts.tolist())) and empty[acts].all(), (use, c, k, len(acts))
            got = legal_of(oracle.widen_mask(words, 225, 1000, oracle.widen_target(c, k) if use else 0, 99, 5))
            assert got.sum() == want and not (got & ~empty).any()
    # the cap: the first moves in move order; then the subset is taken among them
    capped = legal_of(oracle.widen_mask(words, 225, 40, 0, 1, 0))
    assert capped.sum() == 40 and np.array_equal(np.nonzero(capped)[0], np.nonzero(empty)[0][:40])
    both = legal_of(oracle.widen_mask(words, 225, 40, 8, 1, 0))
    assert both.sum() == 8 and not (both & ~capped).any()
    # deterministic in (seed, node); different nodes and seeds choose differently; no move is favoured
    a = legal_of(oracle.widen_mask(words, 225, 0, 8, 7, 3))
    assert np.array_equal(a, legal_of(oracle.widen_mask(words, 225, 0, 8, 7, 3)))
    assert not np.array_equal(a, legal_of(oracle.widen_mask(words, 225, 0, 8, 7, 4)))
    assert not np.array_equal(a, legal_of(oracle.widen_mask(words, 225, 0, 8, 8, 3)))
    counts = np.zeros(225)
    for node in range(3000):
        counts += legal_of(oracle.widen_mask(words, 225, 0, 8, 11, node))
    assert counts[~empty].sum() == 0
    expect = 3000 * 8 / 222
    assert np.abs(counts[empty] - expect).max() < 5 * np.sqrt(expect)


def test_search_restatement_with_widening(oracle):
    """oracle.search_move with progressive widening: every node has at most `target` children, all of them legal
    moves of its position, and a child's position is its parent's plus the move (so a widened parent's other legal
    moves are legal again below it)."""
    rng = np.random.default_rng(6)
    T, spt, R = 2, 8, 30
    games = [[112, 113], [0, 224, 16]]
    pol = rng.dirichlet(np.ones(225) * 0.3, size=(R + 1, T * spt)).astype(np.float32)
    val = (np.round(rng.uniform(-1, 1, (R + 1, T * spt)) * 256) / 256).astype(np.float32)
    tree = oracle.search_move(games, pol[0, :T], None, 0.0, pol[1:], val[1:], spt, T * (1 + R * spt), tt_seed=3,
                              widen=(1000, 8, 12345))
    n = tree["nodes"]
    legal_of = lambda w: np.unpackbits(w.view(np.uint8), bitorder="little")[:225].astype(bool)
    assert n > T
    for node in range(n):
        kids, empty = legal_of(tree["legal_bits"][node]), legal_of(tree["empty_bits"][node])
        assert kids.sum() == min(8, empty.sum()) and not (kids & ~empty).any()
        assert not tree["P"][node, :225][~kids].any()
    child = tree["child_node"][:n, :225]
    for p, a in zip(*np.nonzero(child >= 0)):
        ep, ec = legal_of(tree["empty_bits"][p]), legal_of(tree["empty_bits"][child[p, a]])
        assert legal_of(tree["legal_bits"][p])[a] and ep[a] and not ec[a] and np.array_equal(np.delete(ep, a), np.delete(ec, a))
    assert (tree["N"][:T, :225].sum(1) == spt * R).all() and not tree["VL"].any()


def load_attack_defense_golden():
    """[(board_size, boards int8 [n, S*S], to_move, attack, defense)] from attack_defense_golden.npz; the inputs are
    regenerated from their seeds and checked against the stored checksum."""
    import hashlib
    g = np.load(os.path.join(GOLD, "attack_defense_golden.npz"))
    boards, tm = synth.make_threat_positions(40, 15, seed=77)
    small, small_tm = synth.make_threat_positions(12, 9, seed=78)
    h = hashlib.sha256()
    for a in (boards, tm, small, small_tm):
        h.update(np.ascontiguousarray(a).tobytes())
    assert h.hexdigest() == str(g["inputs_sha256"]), "synth.make_threat_positions changed: regenerate the fixture"
    assert bool(g["integral"]) and int(g["compute_planes_nonzero"]) == 0
    return [(15, boards, tm, g["attack15"].astype(np.float32), g["defense15"].astype(np.float32)),
            (9, small, small_tm, g["attack9"].astype(np.float32), g["defense9"].astype(np.float32))]


def test_attack_defense_matches_reference_golden(oracle):
    """The threat-window restatement against GomokuAttackDefenseModule::compute_bonuses (stone placed) on boards
    with planted threes and fours; the fixture also records that compute_planes itself returned nothing but
    zeros on 24 played games."""
    for S, boards, tm, att, dfn in load_attack_defense_golden():
        a, d = oracle.gomoku_attack_defense(boards, tm, S, stone_placed=True)
        assert np.array_equal(a, att) and np.array_equal(d, dfn)
        a0, d0 = oracle.gomoku_attack_defense(boards, tm, S, stone_placed=False)
        assert not a0.any() and not d0.any()
    # a known answer: three in a row with open ends is one window of 5 and two of 6
    board = np.zeros(225, np.int8)
    board[[7 * 15 + 5, 7 * 15 + 6, 7 * 15 + 7]] = 1
    assert oracle.gomoku_threats(board, 1) == 1 + 2 + 0 and oracle.gomoku_threats(board, 2) == 0


def test_attack_defense_live_against_the_reference_module(oracle):
    _need_ref(oracle, "tree")
    boards, tm = synth.make_threat_positions(16, 15, seed=5)
    ra, rd = oracle.gomoku_attack_defense(boards, tm, 15, True)
    for b in range(len(boards)):
        a, d = oracle.ref_attack_defense_bonuses(boards[b], int(tm[b]), 15)
        assert np.array_equal(a, ra[b]) and np.array_equal(d, rd[b])
    games, _, _, _ = synth.make_gomoku_games(6, 15, seed=9, max_moves=40)
    for g in games:
        a, d = oracle.ref_attack_defense_planes(g, 15)
        assert not a.any() and not d.any()


def load_omok_golden(name="omok_golden.npz"):
    """(games, legal [n, 225] bool) from omok_golden.npz / renju_golden.npz: the legal moves of the reference's
    GomokuState constructed with use_omok / use_renju, after seeded play."""
    g = np.load(os.path.join(GOLD, name))
    ptr = g["row_ptr"]
    games = [g["moves"][ptr[i]:ptr[i + 1]].astype(np.int64).tolist() for i in range(len(ptr) - 1)]
    legal = np.unpackbits(g["legal_bits"])[:len(games) * 225].reshape(len(games), 225).astype(bool)
    assert int(g["forbidden_cells"]) >= 40
    return games, legal


def _legal_of(words, n=225):
    return np.unpackbits(np.ascontiguousarray(words).view(np.uint8), bitorder="little")[:n].astype(bool)


def test_omok_legal_moves_match_reference_golden(oracle):
    """BLACK's forbidden moves under Omok (six or more in a row, open threes in two directions) against the legal
    moves of the reference's GomokuState constructed with use_omok, and two known answers."""
    games, legal = load_omok_golden()
    forbidden = 0
    for mv, want in zip(games, legal):
        got = _legal_of(oracle.gomoku_legal_mask(mv, 15, rules=1))
        assert np.array_equal(got, want), mv
        empty = np.ones(225, bool)
        empty[mv] = False
        forbidden += int((empty & ~got).sum())
        assert np.array_equal(_legal_of(oracle.gomoku_legal_mask(mv, 15, rules=0)), empty)
    assert forbidden >= 40
    # a cross of two open twos: the centre makes two open threes; black to move (white's stones far away)
    black = [7 * 15 + 6, 7 * 15 + 8, 6 * 15 + 7, 8 * 15 + 7]
    white = [0, 14, 210, 224]
    mv = [m for pair in zip(black, white) for m in pair]
    assert not _legal_of(oracle.gomoku_legal_mask(mv, 15, rules=1))[7 * 15 + 7]
    assert _legal_of(oracle.gomoku_legal_mask(mv, 15, rules=0))[7 * 15 + 7]
    # five with a gap: the gap would make six
    black = [7 * 15 + c for c in (2, 3, 4, 6, 7)]
    white = [0, 14, 210, 224, 1]
    mv = [m for pair in zip(black, white) for m in pair]
    assert not _legal_of(oracle.gomoku_legal_mask(mv, 15, rules=1))[7 * 15 + 5]
    # with WHITE to move nothing is forbidden
    assert _legal_of(oracle.gomoku_legal_mask(mv + [7 * 15 + 10], 15, rules=1))[7 * 15 + 5]


def test_omok_legal_moves_live_against_gomokustate(oracle):
    _need_ref(oracle, "tree")
    games, _ = load_omok_golden()
    for mv in games[:24]:
        for cut in (len(mv), len(mv) - 1, len(mv) // 2):
            want = oracle.ref_gomoku_legal_moves(mv[:cut], 15, renju=False, omok=True)
            assert want is not None and np.array_equal(_legal_of(oracle.gomoku_legal_mask(mv[:cut], 15, rules=1)), want)


def test_renju_legal_moves_match_reference_golden(oracle):
    """BLACK's forbidden moves under Renju (overline, double four, double three, as the reference defines them)
    against the legal moves of the reference's GomokuState constructed with use_renju; the recursion limit of the
    restatement is never reached; and the win rule: BLACK needs exactly five."""
    import ctypes as C
    games, legal = load_omok_golden("renju_golden.npz")
    forbidden = 0
    for mv, want in zip(games, legal):
        got = _legal_of(oracle.gomoku_legal_mask(mv, 15, rules=2))
        assert np.array_equal(got, want), mv
        empty = np.ones(225, bool)
        empty[mv] = False
        forbidden += int((empty & ~got).sum())
    assert forbidden >= 500
    L = oracle.lib()
    L.oracle_renju_depth_hits.restype = C.c_int
    assert L.oracle_renju_depth_hits() == 0
    # the gap of X X X _ X X would make six: forbidden under Renju; an exact five is allowed
    black = [7 * 15 + c for c in (2, 3, 4, 6, 7)]
    white = [0, 14, 210, 224, 1]
    mv = [m for pair in zip(black, white) for m in pair]
    assert not _legal_of(oracle.gomoku_legal_mask(mv, 15, rules=2))[7 * 15 + 5]
    assert oracle.gomoku_result(mv + [7 * 15 + 5], 15, rules=2) == 0 and oracle.gomoku_result(mv + [7 * 15 + 5], 15, rules=0) == 1
    black = [7 * 15 + c for c in (3, 4, 6, 7)]
    mv = [m for pair in zip(black, white[:4]) for m in pair]
    assert _legal_of(oracle.gomoku_legal_mask(mv, 15, rules=2))[7 * 15 + 5]
    assert oracle.gomoku_result(mv + [7 * 15 + 5], 15, rules=2) == 1
    # WHITE wins with six under Renju
    white6 = [7 * 15 + c for c in (2, 3, 4, 6, 7, 5)]
    black6 = [0, 14, 210, 224, 1, 16]
    assert oracle.gomoku_result([m for pair in zip(black6, white6) for m in pair], 15, rules=2) == 2


def test_renju_live_against_gomokustate(oracle):
    _need_ref(oracle, "tree")
    games, _ = load_omok_golden("renju_golden.npz")
    for mv in games[:24]:
        for cut in (len(mv), len(mv) - 1, len(mv) // 2):
            want = oracle.ref_gomoku_legal_moves(mv[:cut], 15, renju=True, omok=False)
            assert want is not None and np.array_equal(_legal_of(oracle.gomoku_legal_mask(mv[:cut], 15, rules=2)), want)
    black = [7 * 15 + c for c in (3, 4, 6, 7)]
    white = [0, 14, 210, 224]
    mv = [m for pair in zip(black, white) for m in pair] + [7 * 15 + 5]
    assert oracle.ref_gomoku_result_variant(mv, 15, renju=True) == oracle.gomoku_result(mv, 15, rules=2) == 1
    white6 = [7 * 15 + c for c in (2, 3, 4, 6, 7, 5)]
    black6 = [0, 14, 210, 224, 1, 16]
    mv = [m for pair in zip(black6, white6) for m in pair]
    assert oracle.ref_gomoku_result_variant(mv, 15, renju=True) == oracle.gomoku_result(mv, 15, rules=2) == 2


def test_rule_cases_of_the_reference_unit_tests(oracle):
    """The known answers of the reference's own rule tests (tests/games/gomoku/gomoku_test.cpp:372-452 Omok,
    :485-637 Renju): stone sets with BLACK to move and the cell whose legality the test asserts."""
    import ctypes as C
    L = oracle.lib()
    i8 = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
    L.oracle_omok_forbidden.argtypes = [i8, C.c_int, C.c_int]
    L.oracle_renju_forbidden.argtypes = [i8, C.c_int, C.c_int]

    def board(black, white):
        b = np.zeros(225, np.int8)
        for r, c in black:
            b[r * 15 + c] = 1
        for r, c in white:
            b[r * 15 + c] = 2
        return b
    omok = [  # OmokDoubleThree{PlusShape, XShape, Corner_NE, Corner_SW, TT_W, TT_N, TT_E, TT_S}: all forbidden
        ([(2, 3), (3, 2), (3, 4), (4, 3)], (3, 3)), ([(2, 2), (2, 4), (4, 2), (4, 4)], (3, 3)),
        ([(1, 2), (3, 2), (2, 1), (2, 3)], (2, 2)), ([(2, 2), (2, 3), (1, 1), (3, 1)], (2, 1)),
        ([(3, 1), (3, 2), (2, 3), (4, 3)], (3, 3)), ([(1, 3), (2, 3), (3, 2), (3, 4)], (3, 3)),
        ([(3, 5), (3, 4), (2, 3), (4, 3)], (3, 3)), ([(5, 3), (4, 3), (3, 2), (3, 4)], (3, 3))]
    for black, (r, c) in omok:
        assert L.oracle_omok_forbidden(board(black, [(8, 8)]), 15, r * 15 + c) == 1, (black, r, c)
    renju = [  # (black, white, cell, forbidden): RenjuOverlineBlack, DoubleFourBlack, SimpleDoubleThreeBlackForbidden,
        #        DoubleThreeException_a, DoubleThreeException_b
        ([(7, 3), (7, 4), (7, 5), (7, 6), (7, 8)], [(0, 0)], (7, 7), 1),
        ([(2, 3), (2, 4), (2, 6), (4, 2), (4, 3), (4, 5), (4, 6)], [(7, 7)], (2, 5), 1),
        ([(2, 3), (4, 5), (2, 5), (4, 3)], [(7, 7)], (3, 4), 1),
        ([(2, 2), (2, 4), (4, 1), (5, 2)], [(7, 7)], (3, 3), 0),
        ([(5, 7), (6, 7), (8, 7), (7, 5), (7, 6), (7, 8)], [(4, 7), (7, 4), (7, 9)], (7, 7), 0)]
    for black, white, (r, c), want in renju:
        assert L.oracle_renju_forbidden(board(black, white), 15, r * 15 + c) == want, (black, r, c)
    # RenjuOverlineWhite / RenjuDoubleFourWhiteAllowed: WHITE is never restricted, and its six in a row wins
    white6 = [7 * 15 + c for c in (3, 4, 5, 7, 8, 6)]
    black6 = [0, 14, 210, 224, 1, 16]
    assert oracle.gomoku_result([m for pair in zip(black6, white6) for m in pair], 15, rules=2) == 2
