"""Generates the golden fixtures in this directory from the reference
project's own classes (oracle/_ref, built by `make -C oracle ref` in a
container where the reference checkout is present).

    python tests/golden/make_golden.py

Inputs come from omoknuni_small_b200.synth with fixed seeds; the fixtures store
the inputs' checksums and the reference's outputs:
  select_golden.npz  MCTSNode::selectChild + applyVirtualLoss + revertVirtualLoss
  encode_golden.npz  GomokuState::getEnhancedTensorRepresentation (bit-packed)
  result_golden.npz  GomokuState::isTerminal / getGameResult after one more move
  go_golden.npz      GoState (stones, ko point, side to move, legal cells) and its
                     getEnhancedTensorRepresentation planes after seeded random
                     legal play, 9x9 and 19x19 (`python make_golden.py go` makes
                     only this one)
  chess_golden.npz   ChessState (pieces, side to move, castling, en passant, clocks,
                     legal destinations) and its getEnhancedTensorRepresentation
                     planes after seeded random legal play (`make_golden.py chess`)
  attack_defense_golden.npz  GomokuAttackDefenseModule: compute_planes on played games (all zero) and
                     compute_bonuses with the stone placed on boards with planted threes and
                     fours (`make_golden.py attack_defense`)
  omok_golden.npz    GomokuState(use_omok) legal moves after seeded play that keeps to the centre, so that
                     six-in-a-row and double-three cells occur (`make_golden.py omok`)
  renju_golden.npz   the same for GomokuState(use_renju): overlines, double fours, double threes, and the
                     state's result (BLACK wins with exactly five only) (`make_golden.py renju`)
  net_golden.npz     ResNetModel::forward (log-softmax policy, value): (a) a tiny
                     model with the reference's own libtorch default
                     initialisation, its weights stored here rounded to fp16
                     (the rounded values are what the reference ran with);
                     (b) the 15x15 / 10-block model with seeded weights set by
                     name (regenerated from the seed, checked by checksum).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from omoknuni_small_b200 import synth  # noqa: E402
from oracle import capi  # noqa: E402


def checksum(*arrays):
    import hashlib
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def make_select():
    out = {}
    for tag, n_nodes, nc, seed in (("g225", 256, 225, 7), ("c4672", 8, 4672, 11), ("n3", 64, 3, 5)):
        t = synth.make_selection_tree(n_nodes, nc, seed=seed)
        sel, vl_apply, vl_revert, _ = capi.ref_select(t, c_puct=1.5, vl_value=3)
        out[tag + "_sel"] = sel
        out[tag + "_vl_after_apply"] = vl_apply
        out[tag + "_vl_after_revert"] = vl_revert
        out[tag + "_inputs_sha256"] = checksum(t["N"], t["W"], t["P"], t["VL"], t["legal_bits"], t["node_visits"])
        out[tag + "_shape"] = np.array([n_nodes, nc, seed])
    np.savez_compressed(os.path.join(HERE, "select_golden.npz"), **out)


def make_encode():
    games, hist, nh, tm = synth.make_gomoku_games(48, 15, seed=2024, max_moves=60)
    ref, _ = capi.ref_gomoku_encode_batch(games, 15)
    flat = np.concatenate(games) if sum(map(len, games)) else np.zeros(0, np.int32)
    ptr = np.cumsum([0] + [len(g) for g in games])
    np.savez_compressed(os.path.join(HERE, "encode_golden.npz"), moves=flat.astype(np.int16), row_ptr=ptr,
                        to_move=tm, planes_bits=np.packbits(ref.astype(bool)), planes_shape=np.array(ref.shape),
                        planes_is_binary=np.array(bool(np.isin(ref, (0.0, 1.0)).all())))


def make_net():
    out = {}
    # (a) the reference module as its constructor leaves it (libtorch default initialisation
    #     after torch::manual_seed), tiny shape so that the weights fit in a fixture; every
    #     weight is rounded to fp16 and pushed back so that fixture and outputs agree exactly
    net = capi.RefNet(17, 5, 1, 64, 25, seed=1234)
    x = synth.make_stone_planes(8, 5, 17, seed=77, max_stones=12)
    for name, arr in net.state().items():
        if "num_batches" in name:
            continue
        r = arr.astype(np.float16)
        net.set(name, r.astype(np.float32))
        out["a_w_" + name] = r
    lp, v, _ = net.forward(x)
    out["a_logp"], out["a_value"], out["a_x_bits"], out["a_x_shape"] = lp, v, np.packbits(x.astype(bool)), np.array(x.shape)
    out["a_cfg"] = np.array([17, 5, 1, 64, 25, 32, 32])
    # (b) benchmark-shaped Gomoku network (15x15, 10 blocks, reference 32/32 heads), seeded
    #     weights set by name on the reference module, random BatchNorm statistics
    shapes = synth.net_tensor_shapes(15, 17, 64, 10, 225, 32, 32)
    w = synth.make_weights(shapes, seed=42, init="torch_default", bn="random")
    net = capi.RefNet(17, 15, 10, 64, 225, seed=0)
    for k, a in w.items():
        net.set(k, a)
    x = synth.make_stone_planes(8, 15, 17, seed=1000)
    lp, v, _ = net.forward(x)
    out["b_logp"], out["b_value"] = lp, v
    out["b_weights_sha256"] = checksum(*[w[k] for k, _ in shapes])
    out["b_x_sha256"] = checksum(x)
    np.savez_compressed(os.path.join(HERE, "net_golden.npz"), **out)


def make_results():
    """Game results of the reference's GomokuState for unfinished games extended by one move."""
    rng = np.random.default_rng(5)
    games, _, _, _ = synth.make_gomoku_games(120, 15, seed=606, max_moves=140)
    flat, ptr, res = [], [0], []
    for g in games:
        occ = set(int(x) for x in g)
        for a in rng.permutation(225)[:12]:
            if int(a) in occ:
                continue
            mv = [int(x) for x in g] + [int(a)]
            flat += mv
            ptr.append(len(flat))
            res.append(capi.ref_gomoku_result(mv))
    np.savez_compressed(os.path.join(HERE, "result_golden.npz"), moves=np.asarray(flat, np.int16),
                        row_ptr=np.asarray(ptr, np.int64), result=np.asarray(res, np.int8))


def make_go():
    """Positions of the reference's GoState with the planes its encoder gives for them."""
    out = {}
    for tag, S, n, max_moves, seed in (("s9", 9, 48, 110, 909), ("s19", 19, 6, 260, 919)):
        gs = capi.random_go_games(n, S, seed=seed, max_moves=max_moves)
        out[tag + "_stones"] = np.stack([g["stones"] for g in gs]).astype(np.int8)
        out[tag + "_ko"] = np.array([g["ko_point"] for g in gs], np.int32)
        out[tag + "_to_move"] = np.array([g["to_move"] for g in gs], np.uint8)
        out[tag + "_legal"] = np.packbits(np.stack([g["legal"] for g in gs]).reshape(n, -1), axis=1)
        out[tag + "_planes"] = np.stack([g["planes"] for g in gs]).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "go_golden.npz"), **out)


def make_chess():
    pieces, meta, legal, planes = capi.ref_chess_positions(160, seed=64, max_plies=140)
    np.savez_compressed(os.path.join(HERE, "chess_golden.npz"), pieces=pieces, meta=meta, legal_to=legal,
                        planes=planes)


def make_attack_defense():
    boards, to_move = synth.make_threat_positions(40, 15, seed=77)
    att = np.zeros(boards.shape, np.float32)
    dfn = np.zeros(boards.shape, np.float32)
    for b in range(len(boards)):
        att[b], dfn[b] = capi.ref_attack_defense_bonuses(boards[b], int(to_move[b]), 15)
    small, small_tm = synth.make_threat_positions(12, 9, seed=78)
    att9 = np.zeros(small.shape, np.float32)
    dfn9 = np.zeros(small.shape, np.float32)
    for b in range(len(small)):
        att9[b], dfn9[b] = capi.ref_attack_defense_bonuses(small[b], int(small_tm[b]), 9)
    games, _, _, _ = synth.make_gomoku_games(24, 15, seed=79, max_moves=60)
    planes_nonzero = 0
    for g in games:
        a, d = capi.ref_attack_defense_planes(g, 15)
        planes_nonzero += int(np.count_nonzero(a)) + int(np.count_nonzero(d))
    np.savez_compressed(os.path.join(HERE, "attack_defense_golden.npz"), inputs_sha256=checksum(boards, to_move, small, small_tm),
                        attack15=att.astype(np.int8), defense15=dfn.astype(np.int8), attack9=att9.astype(np.int8),
                        defense9=dfn9.astype(np.int8), integral=np.array(bool((att == np.rint(att)).all() and (dfn == np.rint(dfn)).all())),
                        compute_planes_nonzero=np.array(planes_nonzero))


def make_variant(name, renju, omok, seed):
    rng = np.random.default_rng(seed)
    games, masks, forbidden = [], [], 0
    while len(games) < 64:
        moves = []
        for _ in range(int(rng.integers(8, 70))):
            legal = capi.ref_gomoku_legal_moves(moves, 15, renju, omok)
            cand = np.nonzero(legal)[0]
            if len(cand) == 0 or (moves and capi.ref_gomoku_result(moves, 15) != 0):
                break
            near = [a for a in cand if abs(a // 15 - 7) <= 3 and abs(a % 15 - 7) <= 3]
            moves.append(int(rng.choice(near if near and rng.random() < 0.85 else cand)))
        if moves and capi.ref_gomoku_result(moves, 15) != 0:
            moves.pop()
        legal = capi.ref_gomoku_legal_moves(moves, 15, renju, omok)
        empty = np.ones(225, bool)
        empty[moves] = False
        n_forbidden = int((empty & ~legal).sum())
        if n_forbidden == 0 and len(games) % 4 != 3:      # keep mostly positions where the rule bites
            continue
        forbidden += n_forbidden
        games.append(moves)
        masks.append(legal)
    flat = np.concatenate([np.asarray(g, np.int16) for g in games])
    ptr = np.cumsum([0] + [len(g) for g in games])
    np.savez_compressed(os.path.join(HERE, name), moves=flat, row_ptr=ptr, legal_bits=np.packbits(np.array(masks)),
                        forbidden_cells=np.array(forbidden))


def make_omok():
    make_variant("omok_golden.npz", False, True, 2025)


def make_renju():
    make_variant("renju_golden.npz", True, False, 2026)


if __name__ == "__main__":
    if not (capi.have_ref_tree() and capi.have_ref_net()):
        sys.exit("oracle/_ref is not built: run `make -C oracle ref` where the reference checkout exists")
    if sys.argv[1:] == ["go"]:
        make_go()
        sys.exit(0)
    if sys.argv[1:] == ["chess"]:
        make_chess()
        sys.exit(0)
    if sys.argv[1:] == ["omok"]:
        make_omok()
        sys.exit(0)
    if sys.argv[1:] == ["renju"]:
        make_renju()
        sys.exit(0)
    if sys.argv[1:] == ["attack_defense"]:
        make_attack_defense()
        sys.exit(0)
    make_select()
    make_encode()
    make_net()
    make_results()
    make_go()
    make_chess()
    make_attack_defense()
    make_omok()
    make_renju()
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))
