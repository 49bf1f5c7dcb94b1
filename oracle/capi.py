"""ctypes bindings of the oracle libraries (test infrastructure).

liboracle.so       plain-C restatement (oracle/oracle.c), always buildable.
_ref/libref_tree.so  the reference's MCTSNode / GomokuState compiled from its
                     own sources (oracle/ref_shim_tree.cpp), when present.
_ref/libref_net.so   the reference's ResNetModel on libtorch CPU
                     (oracle/ref_shim_net.cpp), when present.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_i32 = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_f32 = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u32 = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_i16 = np.ctypeslib.ndpointer(np.int16, flags="C_CONTIGUOUS")
_u8 = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i64 = np.ctypeslib.ndpointer(np.int64, flags="C_CONTIGUOUS")


def _opt(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def build():
    """Compile liboracle.so (and oracle/_ref when the reference checkout exists)."""
    subprocess.run(["make", "-C", _HERE, "-j8"], check=True, stdout=subprocess.DEVNULL)


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, stdout=subprocess.DEVNULL)
        L = C.CDLL(path)
        L.oracle_puct_select.argtypes = [_i32, _f32, _f32, _i32, _u32, _i32, C.c_int, C.c_int, C.c_int,
                                         C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_int, _i32, C.c_int]
        L.oracle_vl_apply.argtypes = [_i32, C.c_int, C.c_void_p, _i32, C.c_int, C.c_int]
        L.oracle_vl_revert.argtypes = [_i32, C.c_int, C.c_void_p, _i32, C.c_int, C.c_int]
        L.oracle_vl_ops.argtypes = [C.c_int, _i32, C.c_int, _i32]
        L.oracle_backup.argtypes = [_i32, _f32, _i32, _i32, C.c_void_p, C.c_int, _i32, _i32, _f32, C.c_int,
                                    C.c_int, C.c_int]
        L.oracle_set_priors.argtypes = [_f32, _u32, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, _f32,
                                        C.c_int, C.c_void_p]
        L.oracle_traverse.argtypes = [_i32, _f32, _f32, _i32, _u32, _i32, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                      C.c_int, _i32, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, _i32, _i32]
        L.oracle_gomoku_encode_batch.argtypes = [_i16, _u8, _u8, C.c_int, C.c_int, C.c_int, _f32, C.c_int]
        L.oracle_gomoku_result.argtypes = [_i16, C.c_int, C.c_int]
        _lib = L
    return _lib


# ---- plain-C restatement -----------------------------------------------------
def puct_select(tree, node_ids=None, c_puct=1.5, vl_value=3, apply_vl=False, threads=0):
    """tree: dict of numpy arrays N, W, P, VL [n_nodes, pitch], legal_bits
    [n_nodes, mask_words], node_visits [n_nodes], n_children.  VL is updated in
    place when apply_vl."""
    n_nodes, pitch = tree["N"].shape
    ids = None if node_ids is None else np.ascontiguousarray(node_ids, np.int32)
    n = n_nodes if ids is None else len(ids)
    sel = np.empty(n, np.int32)
    lib().oracle_puct_select(tree["N"], tree["W"], tree["P"], tree["VL"], tree["legal_bits"],
                             tree["node_visits"], tree["n_children"], pitch, tree["legal_bits"].shape[1],
                             _opt(ids), n, c_puct, vl_value, int(apply_vl), sel, threads)
    return sel


def vl_apply(tree, sel, vl_value, node_ids=None):
    ids = None if node_ids is None else np.ascontiguousarray(node_ids, np.int32)
    lib().oracle_vl_apply(tree["VL"], tree["VL"].shape[1], _opt(ids), np.ascontiguousarray(sel, np.int32),
                          len(sel), vl_value)


def vl_revert(tree, sel, vl_value, node_ids=None):
    ids = None if node_ids is None else np.ascontiguousarray(node_ids, np.int32)
    lib().oracle_vl_revert(tree["VL"], tree["VL"].shape[1], _opt(ids), np.ascontiguousarray(sel, np.int32),
                           len(sel), vl_value)


def vl_ops(initial, ops):
    ops = np.ascontiguousarray(ops, np.int32)
    out = np.empty(len(ops), np.int32)
    lib().oracle_vl_ops(initial, ops, len(ops), out)
    return out


def backup(tree, paths, path_len, leaf_values, vl_value):
    paths = np.ascontiguousarray(paths, np.int32)
    n, max_depth, _ = paths.shape
    cn = tree.get("child_node")
    lib().oracle_backup(tree["N"], tree["W"], tree["VL"], tree["node_visits"], _opt(cn), tree["N"].shape[1],
                        paths, np.ascontiguousarray(path_len, np.int32),
                        np.ascontiguousarray(leaf_values, np.float32), n, max_depth, vl_value)


def set_priors(tree, node_ids, policy, slot_action=None):
    ids = None if node_ids is None else np.ascontiguousarray(node_ids, np.int32)
    policy = np.ascontiguousarray(policy, np.float32)
    sa = None if slot_action is None else np.ascontiguousarray(slot_action, np.int32)
    lib().oracle_set_priors(tree["P"], tree["legal_bits"], tree["n_children"], tree["P"].shape[1],
                            tree["legal_bits"].shape[1], _opt(ids), policy.shape[0], policy, policy.shape[1],
                            _opt(sa))


def traverse(tree, roots, sims_per_tree, c_puct, vl_value, max_depth):
    roots = np.ascontiguousarray(roots, np.int32)
    n = len(roots) * sims_per_tree
    paths = np.zeros((n, max_depth, 2), np.int32)
    plen = np.zeros(n, np.int32)
    n_nodes, pitch = tree["N"].shape
    lib().oracle_traverse(tree["N"], tree["W"], tree["P"], tree["VL"], tree["legal_bits"], tree["node_visits"],
                          _opt(tree.get("child_node")), n_nodes, tree["n_children"], pitch,
                          tree["legal_bits"].shape[1], roots, len(roots), sims_per_tree, c_puct, vl_value,
                          max_depth, paths, plen)
    return paths, plen


def gomoku_encode(history, n_hist, to_move, board_size=15, planes=19, threads=0):
    """history [B,16] int16 (k-th most recent move), n_hist [B] u8, to_move [B] u8
    -> planes [B, planes, S, S] fp32."""
    history = np.ascontiguousarray(history, np.int16)
    B = history.shape[0]
    out = np.empty((B, planes, board_size, board_size), np.float32)
    lib().oracle_gomoku_encode_batch(history, np.ascontiguousarray(n_hist, np.uint8),
                                     np.ascontiguousarray(to_move, np.uint8), B, board_size, planes, out, threads)
    return out


def gomoku_planes3(stones, to_move):
    """stones [B,S,S] int8 (0 empty, 1 black, 2 white), to_move [B] u8 -> planes [B, 3, S, S] fp32."""
    stones = np.ascontiguousarray(stones, np.int8)
    B, S = stones.shape[0], stones.shape[1]
    out = np.empty((B, 3, S, S), np.float32)
    lib().oracle_gomoku_planes3_batch(stones.ctypes.data_as(C.c_void_p), np.ascontiguousarray(to_move, np.uint8).ctypes.data_as(C.c_void_p),
                                      B, S, out.ctypes.data_as(C.c_void_p))
    return out


def stones_from_moves(moves, board_size):
    """Board of a Gomoku game given as its move list (black moves first): [S,S] int8 and the side to move."""
    st = np.zeros(board_size * board_size, np.int8)
    for i, m in enumerate(moves):
        st[int(m)] = 1 + (i & 1)
    return st.reshape(board_size, board_size), 1 + (len(moves) & 1)


def go_encode(stones, ko_point, to_move, legal):
    """stones [B,S,S] int8 (0 empty, 1 black, 2 white), ko_point [B] int32 (-1 none), to_move [B] u8,
    legal [B,S,S] u8 -> planes [B, 10, S, S] fp32."""
    stones = np.ascontiguousarray(stones, np.int8)
    B, S = stones.shape[0], stones.shape[1]
    out = np.empty((B, 10, S, S), np.float32)
    lib().oracle_go_encode_batch(stones.ctypes.data_as(C.c_void_p), np.ascontiguousarray(ko_point, np.int32).ctypes.data_as(C.c_void_p),
                                 np.ascontiguousarray(to_move, np.uint8).ctypes.data_as(C.c_void_p),
                                 np.ascontiguousarray(legal, np.uint8).ctypes.data_as(C.c_void_p), B, S,
                                 out.ctypes.data_as(C.c_void_p))
    return out


def chess_encode(pieces, meta, legal_to):
    """pieces [B,64] int8, meta [B,6] int32, legal_to [B,2] uint32 -> planes [B, 20, 8, 8] fp32
    (field meanings: oracle_chess_encode in oracle.c)."""
    pieces = np.ascontiguousarray(pieces, np.int8)
    B = pieces.shape[0]
    out = np.empty((B, 20, 8, 8), np.float32)
    lib().oracle_chess_encode_batch(pieces.ctypes.data_as(C.c_void_p), np.ascontiguousarray(meta, np.int32).ctypes.data_as(C.c_void_p),
                                    np.ascontiguousarray(legal_to, np.uint32).ctypes.data_as(C.c_void_p), B,
                                    out.ctypes.data_as(C.c_void_p))
    return out


def zobrist_keys(seed):
    """The 451 Zobrist keys of a search created with `seed` (splitmix64 stream): [0,225) BLACK stones,
    [225,450) WHITE stones, [450] side to move."""
    M = (1 << 64) - 1
    x = (seed ^ 0xD1B54A32D192ED03) & M
    out = np.empty(451, np.uint64)
    for i in range(451):
        x = (x + 0x9E3779B97F4A7C15) & M
        v = x
        v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & M
        v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & M
        out[i] = v ^ (v >> 31)
    return out


def root_hash(moves, tree_index, zobrist):
    """Key of a root position: its stones, the side to move, and the per-game salt that keeps the
    games of one search from sharing nodes."""
    M = (1 << 64) - 1
    h = 0
    for i, m in enumerate(moves):
        h ^= int(zobrist[(i & 1) * 225 + int(m)])
    if len(moves) & 1:
        h ^= int(zobrist[450])
    return h ^ ((0x9E3779B97F4A7C15 * (tree_index + 1)) & M)


def widen_mask(empty_words, n_children, max_children, target, seed, node_id):
    """The children a node gets out of its legal moves (oracle_widen_mask in oracle.c)."""
    e = np.ascontiguousarray(empty_words, np.uint32)
    out = np.zeros_like(e)
    L = lib()
    L.oracle_widen_mask.argtypes = [_u32, _u32, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_int]
    L.oracle_widen_mask(e, out, n_children, len(e), max_children, target, seed, node_id)
    return out


def widen_target(c, k, visits=0):
    L = lib()
    L.oracle_widen_target.argtypes = [C.c_float, C.c_float, C.c_int]
    L.oracle_widen_target.restype = C.c_int
    return int(L.oracle_widen_target(c, k, visits))


def gomoku_legal_mask(moves, board_size=15, rules=0):
    """Legal moves of the position after `moves` as mask words (oracle_gomoku_legal_mask in oracle.c); rules 1 = Omok."""
    mv = np.ascontiguousarray(moves, np.int16)
    mw = (board_size * board_size + 31) // 32
    out = np.zeros(mw, np.uint32)
    L = lib()
    L.oracle_gomoku_legal_mask.argtypes = [_i16, C.c_int, C.c_int, C.c_int, _u32, C.c_int]
    L.oracle_gomoku_legal_mask(mv, len(mv), board_size, rules, out, mw)
    return out


def search_new_trees(move_lists, max_nodes, n_children=225, widen=None):
    """Edge arrays for a search over the given games: node t is the root of game t (existence mask =
    empty cells), everything else unused.  widen = (max_children, target, seed[, rules]): the empty cells are kept
    in tree["empty_bits"] and the roots' children are the chosen subset of the moves the rules allow."""
    T = len(move_lists)
    pitch, mw = (n_children + 3) // 4 * 4, (n_children + 31) // 32
    t = {"N": np.zeros((max_nodes, pitch), np.int32), "W": np.zeros((max_nodes, pitch), np.float32),
         "P": np.zeros((max_nodes, pitch), np.float32), "VL": np.zeros((max_nodes, pitch), np.int32),
         "child_node": np.full((max_nodes, pitch), -1, np.int32), "legal_bits": np.zeros((max_nodes, mw), np.uint32),
         "node_visits": np.zeros(max_nodes, np.int32), "n_children": n_children, "nodes": T}
    for g, mv in enumerate(move_lists):
        empty = np.ones(n_children, bool)
        empty[np.asarray(mv, np.int64)] = False
        bits = np.zeros(mw * 32, np.uint8)
        bits[:n_children] = empty
        t["legal_bits"][g] = np.packbits(bits.reshape(mw, 32), axis=1, bitorder="little").view(np.uint32).reshape(mw)
    if widen is not None:
        t["empty_bits"] = t["legal_bits"].copy()
        rules = widen[3] if len(widen) > 3 else 0
        for g in range(T):
            legal = gomoku_legal_mask(move_lists[g], 15, rules) if rules else t["empty_bits"][g]
            t["legal_bits"][g] = widen_mask(legal, n_children, widen[0], widen[1], widen[2], g)
    return t


def mix_noise(tree, node_ids, noise, eps):
    ids = np.ascontiguousarray(node_ids, np.int32)
    noise = np.ascontiguousarray(noise, np.float32)
    L = lib()
    L.oracle_mix_noise.argtypes = [_f32, _u32, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, _f32, C.c_float]
    L.oracle_mix_noise(tree["P"], tree["legal_bits"], tree["n_children"], tree["P"].shape[1],
                       tree["legal_bits"].shape[1], _opt(ids), len(ids), noise, eps)


def dirichlet_normalize(gammas):
    g = np.ascontiguousarray(gammas, np.float32).copy()
    L = lib()
    L.oracle_dirichlet_normalize.argtypes = [_f32, C.c_int]
    L.oracle_dirichlet_normalize(g, len(g))
    return g


def search_expand(tree, node_hash, paths, path_len, sims_per_tree, move_lists, policy, value, value_sign,
                  value_quantum, zobrist, board_size=15, widen=None):
    """The expansion step of one round (oracle_search_expand_widen in oracle.c).  tree["nodes"] is the node
    counter and is advanced; node_hash (uint64 [max_nodes]) is None with the table off; widen as in
    search_new_trees.  Returns (leaf_values, terminal flags)."""
    paths = np.ascontiguousarray(paths, np.int32)
    n, max_depth, _ = paths.shape
    T = len(move_lists)
    stride = max(1, max(len(m) for m in move_lists))
    moves = np.full((T, stride), -1, np.int16)
    nm = np.zeros(T, np.int32)
    for g, m in enumerate(move_lists):
        moves[g, :len(m)] = m
        nm[g] = len(m)
    used = np.array([tree["nodes"]], np.int32)
    leaf = np.zeros(n, np.float32)
    term = np.zeros(n, np.int32)
    policy = np.ascontiguousarray(policy, np.float32)
    _u64 = np.ctypeslib.ndpointer(np.uint64, flags="C_CONTIGUOUS")
    L = lib()
    L.oracle_search_expand_widen.argtypes = [_i32, _f32, _f32, _i32, _u32, _i32, _i32, C.c_void_p, _i32, C.c_int, C.c_int, C.c_int,
                                             C.c_int, _i32, _i32, C.c_int, C.c_int, C.c_int, _i16, _i32, C.c_int, C.c_int, _f32,
                                             C.c_int, _f32, C.c_float, C.c_float, _u64, C.c_int, _f32, _i32, C.c_void_p, C.c_int,
                                             C.c_int, C.c_uint64, C.c_int]
    wd = tuple(widen) if widen is not None else (0, 0, 0)
    wd = wd if len(wd) > 3 else wd + (0,)
    L.oracle_search_expand_widen(tree["N"], tree["W"], tree["P"], tree["VL"], tree["legal_bits"], tree["node_visits"],
                           tree["child_node"], _opt(node_hash), used, tree["N"].shape[0], tree["n_children"],
                           tree["N"].shape[1], tree["legal_bits"].shape[1], paths, np.ascontiguousarray(path_len, np.int32),
                           n, max_depth, sims_per_tree, moves, nm, stride, board_size, policy, policy.shape[1],
                           np.ascontiguousarray(value, np.float32), float(value_sign), float(value_quantum),
                           np.ascontiguousarray(zobrist, np.uint64), T, leaf, term,
                           _opt(tree["empty_bits"]) if widen is not None else None, wd[0], wd[1], wd[2], wd[3])
    tree["nodes"] = int(used[0])
    return leaf, term


def search_move(move_lists, root_policy, noise, eps, round_policy, round_value, sims_per_tree, max_nodes, c_puct=1.5,
                vl_value=3, max_depth=64, value_sign=1.0, value_quantum=0.0, tt_seed=None, widen=None):
    """One move of the leaf-parallel search for a group of games, given what the network returned:
    root_policy [T, 225]; round_policy [R, T * sims_per_tree, 225], round_value [R, T * sims_per_tree].
    noise [T, pitch] (or None) is mixed into the root priors with weight eps.  tt_seed: seed of the Zobrist
    keys, None = table off.  Returns the tree dict (tree["nodes"] nodes used) and per-round terminal counts."""
    T = len(move_lists)
    tree = search_new_trees(move_lists, max_nodes, widen=widen)
    roots = np.arange(T, dtype=np.int32)
    set_priors(tree, roots, root_policy)
    if noise is not None and eps > 0:
        mix_noise(tree, roots, noise, eps)
    zob = zobrist_keys(tt_seed if tt_seed is not None else 0)
    node_hash = None
    if tt_seed is not None:
        node_hash = np.zeros(max_nodes, np.uint64)
        for g, mv in enumerate(move_lists):
            node_hash[g] = root_hash(mv, g, zob)
    terminals = 0
    for r in range(len(round_policy)):
        paths, plen = traverse(tree, roots, sims_per_tree, c_puct, vl_value, max_depth)
        leaf, term = search_expand(tree, node_hash, paths, plen, sims_per_tree, move_lists, round_policy[r], round_value[r],
                                   value_sign, value_quantum, zob, widen=widen)
        terminals += int((term > 0).sum())
        backup(tree, paths, plen, leaf, vl_value)
    tree["terminal_leaves"] = terminals
    return tree


def gomoku_threats(board, color, board_size=15):
    """Open-three / open-four window count of a colour (oracle_gomoku_threats in oracle.c)."""
    bd = np.ascontiguousarray(board, np.int8).reshape(-1)
    L = lib()
    L.oracle_gomoku_threats.argtypes = [np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS"), C.c_int, C.c_int]
    return int(L.oracle_gomoku_threats(bd, board_size, color))


def gomoku_attack_defense(stones, to_move, board_size=15, stone_placed=False):
    """(attack, defense) fp32 [B, S*S] for boards int8 [B, S*S] (oracle_gomoku_attack_defense in oracle.c)."""
    st = np.ascontiguousarray(stones, np.int8)
    tm = np.ascontiguousarray(to_move, np.uint8)
    att = np.zeros(st.shape, np.float32)
    dfn = np.zeros(st.shape, np.float32)
    L = lib()
    i8 = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
    u8 = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
    L.oracle_gomoku_attack_defense.argtypes = [i8, u8, C.c_int, C.c_int, C.c_int, _f32, _f32]
    L.oracle_gomoku_attack_defense(st, tm, st.shape[0], board_size, int(stone_placed), att, dfn)
    return att, dfn


def gomoku_result(moves, board_size=15, rules=0):
    """0 ongoing, 1 BLACK won, 2 WHITE won, 3 draw, judged on the last move (rules 2: Renju's exact five for BLACK)."""
    mv = np.ascontiguousarray(moves, np.int16)
    L = lib()
    L.oracle_gomoku_result_rules.argtypes = [_i16, C.c_int, C.c_int, C.c_int]
    return int(L.oracle_gomoku_result_rules(mv, len(mv), board_size, rules))


# ---- the reference's own classes (oracle/_ref) --------------------------------
_ref_tree = None
_ref_net = None


def ref_tree_path():
    return os.path.join(_HERE, "_ref", "libref_tree.so")


def ref_net_path():
    return os.path.join(_HERE, "_ref", "libref_net.so")


def have_ref_tree():
    return os.path.exists(ref_tree_path())


def have_ref_net():
    return os.path.exists(ref_net_path())


def ref_tree():
    global _ref_tree
    if _ref_tree is None:
        L = C.CDLL(ref_tree_path())
        L.ref_select_child.argtypes = [C.c_int, _i32, _f32, _f32, _i32, C.c_int, C.c_float]
        L.ref_select_batch.restype = C.c_double
        L.ref_select_batch.argtypes = [C.c_int, _i64, _i32, _f32, _f32, _i32, _i32, C.c_float, C.c_int, _i32,
                                       C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.ref_vl_ops.argtypes = [C.c_int, _i32, C.c_int, _i32]
        L.ref_backup_path.argtypes = [C.c_int, _i32, _f32, _i32, C.c_float, C.c_int, _f32]
        L.ref_gomoku_encode.argtypes = [C.c_int, _i32, C.c_int, C.c_void_p, C.c_void_p]
        L.ref_gomoku_result.argtypes = [C.c_int, _i32, C.c_int]
        L.ref_gomoku_encode_batch.restype = C.c_double
        L.ref_gomoku_encode_batch.argtypes = [C.c_int, C.c_int, _i64, _i32, _f32, C.c_int]
        if hasattr(L, "ref_go_encode"):
            L.ref_go_encode.argtypes = [C.c_int, C.c_void_p, C.c_int] + [C.c_void_p] * 5
        _ref_tree = L
    return _ref_tree


def compact_rows(tree, node_ids=None):
    """Existing child slots only, as the reference's children_ vectors hold them.
    Returns row_ptr, N, W, P, VL (compacted), slot index of each compacted child,
    node_visits per selected node."""
    n_nodes, pitch = tree["N"].shape
    ids = np.arange(n_nodes) if node_ids is None else np.asarray(node_ids)
    nc = tree["n_children"]
    bits = np.unpackbits(tree["legal_bits"][ids].view(np.uint8), axis=1, bitorder="little")[:, :nc].astype(bool)
    counts = bits.sum(1)
    row_ptr = np.zeros(len(ids) + 1, np.int64)
    np.cumsum(counts, out=row_ptr[1:])
    rows, slots = np.nonzero(bits)
    g = ids[rows]
    return (row_ptr, np.ascontiguousarray(tree["N"][g, slots]), np.ascontiguousarray(tree["W"][g, slots]),
            np.ascontiguousarray(tree["P"][g, slots]), np.ascontiguousarray(tree["VL"][g, slots]),
            slots.astype(np.int32), np.ascontiguousarray(tree["node_visits"][ids]))


def ref_select(tree, node_ids=None, c_puct=1.5, vl_value=3, repeats=1, threads=0):
    """Real MCTSNode::selectChild + applyVirtualLoss + revertVirtualLoss per node.
    Returns (slot per node, VL after apply, VL after revert, seconds)."""
    row_ptr, N, W, P, VL, slots, nv = compact_rows(tree, node_ids)
    n = len(row_ptr) - 1
    sel_c = np.full(n, -1, np.int32)
    a = np.zeros(n, np.int32)
    r = np.zeros(n, np.int32)
    secs = ref_tree().ref_select_batch(n, row_ptr, N, W, P, VL, nv, c_puct, vl_value, sel_c,
                                       a.ctypes.data_as(C.c_void_p), r.ctypes.data_as(C.c_void_p), repeats, threads)
    sel = np.where(sel_c >= 0, slots[np.minimum(row_ptr[:-1] + np.maximum(sel_c, 0), len(slots) - 1)] if len(slots) else -1, -1)
    return sel.astype(np.int32), a, r, secs


def ref_vl_ops(initial, ops):
    ops = np.ascontiguousarray(ops, np.int32)
    out = np.empty(len(ops), np.int32)
    ref_tree().ref_vl_ops(initial, ops, len(ops), out)
    return out


def ref_backup_path(N, W, VL, leaf_value, vl_value):
    N = np.ascontiguousarray(N, np.int32).copy()
    VL = np.ascontiguousarray(VL, np.int32).copy()
    W = np.ascontiguousarray(W, np.float32)
    mean = np.zeros(len(N), np.float32)
    ref_tree().ref_backup_path(len(N), N, W, VL, leaf_value, vl_value, mean)
    return N, VL, mean


def ref_gomoku_planes(moves, board_size=15):
    """Play `moves` on the reference's GomokuState; returns (planes19, planes3, to_move)."""
    mv = np.ascontiguousarray(moves, np.int32)
    p19 = np.zeros((19, board_size, board_size), np.float32)
    p3 = np.zeros((3, board_size, board_size), np.float32)
    tm = ref_tree().ref_gomoku_encode(board_size, mv, len(mv), p19.ctypes.data_as(C.c_void_p),
                                      p3.ctypes.data_as(C.c_void_p))
    if tm < 0:
        raise ValueError("illegal move in list")
    return p19, p3, tm


def ref_expand_gomoku(moves, use_progressive_widening, cpw, kpw, board_size=15):
    """Actions of the children MCTSNode::expand creates at the position after `moves`."""
    mv = np.ascontiguousarray(moves, np.int16)
    out = np.zeros(board_size * board_size, np.int32)
    L = ref_tree()
    L.ref_expand_gomoku.argtypes = [_i16, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, _i32, C.c_int]
    L.ref_expand_gomoku.restype = C.c_int
    n = L.ref_expand_gomoku(mv, len(mv), board_size, int(use_progressive_widening), cpw, kpw, out, len(out))
    assert n >= 0
    return out[:n].copy()


def ref_attack_defense_planes(moves, board_size=15):
    """GomokuAttackDefenseModule::compute_planes on the GomokuState reached by `moves`: (attack, defense) [S*S]."""
    mv = np.ascontiguousarray(moves, np.int16)
    att = np.zeros(board_size * board_size, np.float32)
    dfn = np.zeros_like(att)
    L = ref_tree()
    L.ref_attack_defense_planes.argtypes = [_i16, C.c_int, C.c_int, _f32, _f32]
    L.ref_attack_defense_planes.restype = C.c_int
    assert L.ref_attack_defense_planes(mv, len(mv), board_size, att, dfn) == 0
    return att, dfn


def ref_attack_defense_bonuses(board, player, board_size=15):
    """GomokuAttackDefenseModule::compute_bonuses for every empty cell of `board` (int8 [S*S]) with the player's
    stone placed on it first: (attack, defense) [S*S]."""
    bd = np.ascontiguousarray(board, np.int8).reshape(-1)
    att = np.zeros(board_size * board_size, np.float32)
    dfn = np.zeros_like(att)
    L = ref_tree()
    L.ref_attack_defense_bonuses.argtypes = [np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS"), C.c_int, C.c_int, _f32, _f32]
    L.ref_attack_defense_bonuses.restype = C.c_int
    assert L.ref_attack_defense_bonuses(bd, board_size, player, att, dfn) == 0
    return att, dfn


def ref_gomoku_legal_moves(moves, board_size=15, renju=False, omok=False):
    """GomokuState::getLegalMoves after `moves` on a state constructed with the given variant flags (bool [S*S]);
    None when one of the moves was refused by the state."""
    mv = np.ascontiguousarray(moves, np.int16)
    out = np.zeros(board_size * board_size, np.uint8)
    L = ref_tree()
    L.ref_gomoku_legal_moves.argtypes = [_i16, C.c_int, C.c_int, C.c_int, C.c_int, np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")]
    L.ref_gomoku_legal_moves.restype = C.c_int
    rc = L.ref_gomoku_legal_moves(mv, len(mv), board_size, int(renju), int(omok), out)
    return out.astype(bool) if rc == 0 else None


def ref_gomoku_result(moves, board_size=15):
    mv = np.ascontiguousarray(moves, np.int32)
    return int(ref_tree().ref_gomoku_result(board_size, mv, len(mv)))


def ref_gomoku_result_variant(moves, board_size=15, renju=False, omok=False):
    """The result GomokuState(variant flags) reports after `moves`, played without legality checks."""
    mv = np.ascontiguousarray(moves, np.int32)
    L = ref_tree()
    L.ref_gomoku_result_variant.argtypes = [C.c_int, _i32, C.c_int, C.c_int, C.c_int]
    L.ref_gomoku_result_variant.restype = C.c_int
    return int(L.ref_gomoku_result_variant(board_size, mv, len(mv), int(renju), int(omok)))


def ref_gomoku_encode_batch(move_lists, board_size=15, threads=0):
    row_ptr = np.zeros(len(move_lists) + 1, np.int64)
    np.cumsum([len(m) for m in move_lists], out=row_ptr[1:])
    flat = np.ascontiguousarray(np.concatenate([np.asarray(m, np.int32) for m in move_lists]) if row_ptr[-1] else np.zeros(0, np.int32))
    out = np.zeros((len(move_lists), 19, board_size, board_size), np.float32)
    secs = ref_tree().ref_gomoku_encode_batch(board_size, len(move_lists), row_ptr, flat, out, threads)
    return out, secs


def ref_go_encode(moves, board_size):
    """The reference's GoState after `moves` (cell indices, -1 = pass): dict with stones [S,S] int8,
    ko_point, to_move, legal [S,S] u8 and planes [10,S,S] fp32; None when the move list is illegal."""
    S, S2 = board_size, board_size * board_size
    m = np.ascontiguousarray(moves, np.int32)
    stones = np.zeros(S2, np.int8); legal = np.zeros(S2, np.uint8); planes = np.zeros(10 * S2, np.float32)
    ko = C.c_int32(); tm = C.c_int32()
    n = ref_tree().ref_go_encode(S, m.ctypes.data_as(C.c_void_p), len(m), stones.ctypes.data_as(C.c_void_p), C.byref(ko),
                                 C.byref(tm), legal.ctypes.data_as(C.c_void_p), planes.ctypes.data_as(C.c_void_p))
    if n != 10:
        return None
    return dict(stones=stones.reshape(S, S), ko_point=ko.value, to_move=tm.value, legal=legal.reshape(S, S),
                planes=planes.reshape(10, S, S))


def random_go_games(n_games, board_size, seed, max_moves):
    """Seeded random legal play on the reference's GoState (passes with probability 0.03); one
    position per game, after a random number of moves.  Returns a list of ref_go_encode dicts."""
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n_games):
        target = int(rng.integers(0, max_moves + 1))
        moves = []
        st = ref_go_encode(moves, board_size)
        while len(moves) < target:
            cand = np.flatnonzero(st["legal"].reshape(-1))
            mv = -1 if (len(cand) == 0 or rng.random() < 0.03) else int(rng.choice(cand))
            nxt = ref_go_encode(moves + [mv], board_size)
            if nxt is None:
                break
            moves.append(mv); st = nxt
        out.append(st)
    return out


def ref_chess_positions(n, seed, max_plies):
    """n positions of the reference's ChessState after seeded random legal play: pieces [n,64] int8,
    meta [n,6] int32, legal_to [n,2] uint32, planes [n,20,8,8] fp32.  meta[:,5] (how often the position
    has occurred) is not readable through the reference's public interface: it is recovered from the
    reference's own repetition plane (plane 17 = occurrences / 3)."""
    f = ref_tree().ref_chess_random_encode
    f.restype = C.c_int
    f.argtypes = [C.c_uint64, C.c_int] + [C.c_void_p] * 4
    rng = np.random.default_rng(seed)
    pieces = np.zeros((n, 64), np.int8); meta = np.zeros((n, 6), np.int32); legal = np.zeros((n, 2), np.uint32)
    planes = np.zeros((n, 20, 8, 8), np.float32)
    for i in range(n):
        r = f(int(rng.integers(1, 1 << 40)), int(rng.integers(0, max_plies + 1)), pieces[i].ctypes.data, meta[i].ctypes.data,
              legal[i].ctypes.data, planes[i].ctypes.data)
        assert r >= 0
        meta[i, 5] = int(round(float(planes[i, 17, 0, 0]) * 3))
    return pieces, meta, legal, planes


class RefNet:
    """The reference's alphazero::nn::ResNetModel (libtorch, CPU, fp32)."""

    def __init__(self, in_ch, board, blocks, filters, policy, seed=0):
        global _ref_net
        if _ref_net is None:
            L = C.CDLL(ref_net_path())
            L.ref_net_create.restype = C.c_void_p
            L.ref_net_create.argtypes = [C.c_int] * 5 + [C.c_uint64]
            L.ref_net_destroy.argtypes = [C.c_void_p]
            L.ref_net_names.restype = C.c_int64
            L.ref_net_names.argtypes = [C.c_void_p, C.c_char_p, C.c_int64]
            L.ref_net_get.restype = C.c_int64
            L.ref_net_get.argtypes = [C.c_void_p, C.c_char_p, _f32, C.c_int64]
            L.ref_net_set.restype = C.c_int64
            L.ref_net_set.argtypes = [C.c_void_p, C.c_char_p, _f32, C.c_int64]
            L.ref_net_save.argtypes = [C.c_void_p, C.c_char_p]
            L.ref_net_forward.restype = C.c_double
            L.ref_net_forward.argtypes = [C.c_void_p, _f32, C.c_int, C.c_int, _f32, _f32, C.c_int, C.c_int]
            _ref_net = L
        self.L = _ref_net
        self.board, self.policy, self.in_ch = board, policy or board * board, in_ch
        self.h = self.L.ref_net_create(in_ch, board, blocks, filters, policy, seed)
        if not self.h:
            raise RuntimeError("reference ResNetModel could not be constructed")

    def names(self):
        buf = C.create_string_buffer(1 << 20)
        self.L.ref_net_names(self.h, buf, len(buf))
        return [(l.split()[0], int(l.split()[1])) for l in buf.value.decode().splitlines()]

    def state(self):
        out = {}
        for name, numel in self.names():
            a = np.empty(numel, np.float32)
            self.L.ref_net_get(self.h, name.encode(), a, numel)
            out[name] = a
        return out

    def set(self, name, arr):
        a = np.ascontiguousarray(arr, np.float32).ravel()
        if self.L.ref_net_set(self.h, name.encode(), a, a.size) != a.size:
            raise KeyError(f"{name}: unknown or size mismatch")

    def save(self, path):
        """ResNetModel::save: the reference's checkpoint file."""
        if self.L.ref_net_save(self.h, str(path).encode()) != 0:
            raise RuntimeError("reference save failed")

    def forward(self, x, threads=0, repeats=1):
        """x [B,C,S,S] fp32 -> (log-softmax policy [B,A], value [B], seconds per forward)."""
        x = np.ascontiguousarray(x, np.float32)
        B, Cc = x.shape[:2]
        lp = np.empty((B, self.policy), np.float32)
        v = np.empty(B, np.float32)
        secs = self.L.ref_net_forward(self.h, x, B, Cc, lp, v, threads, repeats)
        if secs < 0:
            raise RuntimeError("reference forward failed")
        return lp, v, secs

    def __del__(self):
        try:
            self.L.ref_net_destroy(self.h)
        except Exception:
            pass
