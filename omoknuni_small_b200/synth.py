"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations: selection trees, Gomoku move histories, input planes
and network weights.  Used by the tests and by bench.py; numpy only.

There is no public dataset behind any of these: the reference project's only
data is its own self-play output, so seeded random positions stand in for it.
"""
import math

import numpy as np


def tree_pitch(n_children):
    return (n_children + 3) // 4 * 4


def tree_mask_words(n_children):
    return (n_children + 31) // 32


def make_selection_tree(n_nodes, n_children=225, seed=7, legal_lo=0.3, legal_hi=1.0, alpha=0.3,
                        vl_max=3, mean_visits=8.0):
    """Edge statistics of `n_nodes` independent nodes in the layout of
    ob200_tree_view: visits N ~ Poisson(mean_visits) int32, W = N * U(-1, 1)
    fp32, a random legal mask holding U(legal_lo, legal_hi) of the child slots,
    priors ~ Dirichlet(alpha) over the legal slots (0 elsewhere), virtual-loss
    counts ~ U{0..vl_max}, node_visits = 1 + sum of legal N.  Illegal and
    padding slots carry random N / W / VL so that masking is exercised."""
    rng = np.random.default_rng(seed)
    pitch, mw = tree_pitch(n_children), tree_mask_words(n_children)
    N = rng.poisson(mean_visits, (n_nodes, pitch)).astype(np.int32)
    W = (N * rng.uniform(-1.0, 1.0, (n_nodes, pitch))).astype(np.float32)
    VL = rng.integers(0, vl_max + 1, (n_nodes, pitch), dtype=np.int32)
    frac = rng.uniform(legal_lo, legal_hi, n_nodes)
    k = np.ceil(frac * n_children).astype(np.int64)
    # random subset of size k per row: rank of a uniform key < k
    keys = rng.random((n_nodes, n_children))
    order = np.argsort(np.argsort(keys, axis=1), axis=1)
    legal = order < k[:, None]
    g = rng.standard_gamma(alpha, (n_nodes, n_children)) * legal
    tot = g.sum(1, keepdims=True)
    tot[tot == 0] = 1.0
    P = np.zeros((n_nodes, pitch), np.float32)
    P[:, :n_children] = (g / tot).astype(np.float32)
    bits = np.zeros((n_nodes, mw * 32), np.uint8)
    bits[:, :n_children] = legal
    legal_bits = np.packbits(bits, axis=1, bitorder="little").view(np.uint32).reshape(n_nodes, mw)
    node_visits = (1 + (N[:, :n_children] * legal).sum(1)).astype(np.int32)
    return {"N": N, "W": W, "P": P, "VL": VL, "legal_bits": np.ascontiguousarray(legal_bits),
            "node_visits": node_visits, "n_children": n_children}


def copy_tree(tree):
    return {k: (v.copy() if isinstance(v, np.ndarray) else v) for k, v in tree.items()}


def selection_bytes_per_node(n_children):
    """Algorithmic bytes of one select + VL apply + VL revert on one node:
    four 4-byte arrays per child slot, one mask bit per slot rounded up to
    32-bit words, node_visits in, selected slot out, and two read-modify-writes
    of one VL word."""
    return n_children * 16 + tree_mask_words(n_children) * 4 + 4 + 4 + 16


def _makes_five(board, S, r, c, colour):
    """True when a stone of `colour` at (r, c) completes five or more in a row."""
    for dr, dc in ((0, 1), (1, 0), (1, 1), (1, -1)):
        run = 1
        for sgn in (1, -1):
            rr, cc = r + sgn * dr, c + sgn * dc
            while 0 <= rr < S and 0 <= cc < S and board[rr, cc] == colour:
                run += 1
                rr += sgn * dr
                cc += sgn * dc
        if run >= 5:
            return True
    return False


def make_gomoku_games(B, board_size=15, seed=1000, max_moves=100):
    """B random, legal, unfinished Gomoku games: k ~ U{0..max_moves} stones on
    distinct random cells, colours alternating from BLACK, skipping any cell
    that would complete five in a row (so no position is terminal).  Returns
    (move_lists, history [B,16] int16 with the k-th most recent move (-1 =
    none), n_hist [B] u8, to_move [B] u8 with 1 = BLACK, 2 = WHITE)."""
    rng = np.random.default_rng(seed)
    S = board_size
    cells = S * S
    move_lists = []
    hist = np.full((B, 16), -1, np.int16)
    n_hist = np.zeros(B, np.uint8)
    to_move = np.ones(B, np.uint8)
    for b in range(B):
        k = int(rng.integers(0, min(max_moves, cells) + 1))
        board = np.zeros((S, S), np.int8)
        mv = []
        for cell in rng.permutation(cells):
            if len(mv) == k:
                break
            colour = 1 + len(mv) % 2
            r, c = divmod(int(cell), S)
            if _makes_five(board, S, r, c, colour):
                continue
            board[r, c] = colour
            mv.append(int(cell))
        mv = np.asarray(mv, np.int32)
        move_lists.append(mv)
        h = mv[::-1][:16]
        hist[b, :len(h)] = h
        n_hist[b] = len(h)
        to_move[b] = 1 if len(mv) % 2 == 0 else 2
    return move_lists, hist, n_hist, to_move


def make_stone_planes(B, board_size=15, channels=17, seed=1000, max_stones=100, history=8):
    """Binary input planes [B, channels, S, S] fp32 as the benchmark
    configuration describes them: `history` cumulative-board planes per player
    (plane 2t = first player's stones t plies ago, 2t+1 = second player's)
    followed by a side-to-move plane; remaining channels (if any) are zero."""
    rng = np.random.default_rng(seed)
    S = board_size
    x = np.zeros((B, channels, S * S), np.float32)
    for b in range(B):
        k = int(rng.integers(0, max_stones + 1))
        cells = rng.permutation(S * S)[:k]
        for t in range(history):
            kk = max(0, k - t)
            if 2 * t < channels:
                x[b, 2 * t, cells[0:kk:2]] = 1.0
            if 2 * t + 1 < channels:
                x[b, 2 * t + 1, cells[1:kk:2]] = 1.0
        if 2 * history < channels:
            x[b, 2 * history, :] = 1.0 if k % 2 == 0 else 0.0
    return x.reshape(B, channels, S, S)


def net_tensor_shapes(board_size, input_channels, filters, blocks, policy_size, policy_head_ch=32,
                      value_head_ch=32, value_hidden=256, policy_planes=False):
    """Names and shapes of the reference module's parameters and buffers
    (reference src/nn/resnet_model.cpp:51-102), in registration order.
    policy_planes: the convolutional policy head (1x1 convolution with bias to
    policy_head_ch planes, no BatchNorm, no FC) instead of the reference's."""
    S2 = board_size * board_size
    out = []

    def bn(prefix, c):
        out.extend([(prefix + ".weight", (c,)), (prefix + ".bias", (c,)),
                    (prefix + ".running_mean", (c,)), (prefix + ".running_var", (c,))])

    out.append(("input_conv.weight", (filters, input_channels, 3, 3)))
    bn("input_bn", filters)
    for i in range(blocks):
        out.append((f"res_blocks.{i}.conv1.weight", (filters, filters, 3, 3)))
        bn(f"res_blocks.{i}.bn1", filters)
        out.append((f"res_blocks.{i}.conv2.weight", (filters, filters, 3, 3)))
        bn(f"res_blocks.{i}.bn2", filters)
    out.append(("policy_conv.weight", (policy_head_ch, filters, 1, 1)))
    if policy_planes:
        out.append(("policy_conv.bias", (policy_head_ch,)))
    else:
        bn("policy_bn", policy_head_ch)
        out.append(("policy_fc.weight", (policy_size, policy_head_ch * S2)))
        out.append(("policy_fc.bias", (policy_size,)))
    out.append(("value_conv.weight", (value_head_ch, filters, 1, 1)))
    bn("value_bn", value_head_ch)
    out.append(("value_fc1.weight", (value_hidden, value_head_ch * S2)))
    out.append(("value_fc1.bias", (value_hidden,)))
    out.append(("value_fc2.weight", (1, value_hidden)))
    out.append(("value_fc2.bias", (1,)))
    return out


def make_weights(shapes, seed=42, init="kaiming_normal", bn="identity"):
    """Seeded fp32 weights for the tensors listed by net_tensor_shapes.

    init = "kaiming_normal": convolutions N(0, sqrt(2 / fan_out)) (fan_out,
        ReLU gain) and linear layers N(0, 0.01) with zero bias, as the
        reference's Python model initialises itself
        (python/alphazero/alphazero_trainer.py:156-168).
    init = "torch_default": U(-1/sqrt(fan_in), 1/sqrt(fan_in)) for weights and
        biases, the distribution libtorch's Conv2d / Linear constructors use,
        which is what the reference's C++ model runs with when nothing is loaded.
    bn = "identity": gamma 1, beta 0, mean 0, var 1.
    bn = "random": gamma U(0.5, 1.5), beta N(0, 0.1), mean N(0, 0.1), var U(0.5, 1.5)
        (exercises the folding)."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in shapes:
        leaf = name.rsplit(".", 1)[-1]
        is_bn = ".bn" in name or name.startswith("input_bn") or name.startswith("policy_bn") or name.startswith("value_bn")
        if is_bn:
            if bn == "identity":
                val = {"weight": 1.0, "bias": 0.0, "running_mean": 0.0, "running_var": 1.0}[leaf]
                w[name] = np.full(shape, val, np.float32)
            else:
                if leaf in ("weight", "running_var"):
                    w[name] = rng.uniform(0.5, 1.5, shape).astype(np.float32)
                else:
                    w[name] = rng.normal(0.0, 0.1, shape).astype(np.float32)
        elif len(shape) == 4:
            co, ci, kh, kw = shape
            if init == "kaiming_normal":
                w[name] = rng.normal(0.0, math.sqrt(2.0 / (co * kh * kw)), shape).astype(np.float32)
            else:
                b = 1.0 / math.sqrt(ci * kh * kw)
                w[name] = rng.uniform(-b, b, shape).astype(np.float32)
        elif len(shape) == 2:
            if init == "kaiming_normal":
                w[name] = rng.normal(0.0, 0.01, shape).astype(np.float32)
            else:
                b = 1.0 / math.sqrt(shape[1])
                w[name] = rng.uniform(-b, b, shape).astype(np.float32)
        else:  # linear bias
            if init == "kaiming_normal":
                w[name] = np.zeros(shape, np.float32)
            else:
                fan_in = dict(shapes)[name.replace(".bias", ".weight")][1]
                b = 1.0 / math.sqrt(fan_in)
                w[name] = rng.uniform(-b, b, shape).astype(np.float32)
    return w


def net_flops_per_eval(board_size, input_channels, filters, blocks, policy_size, policy_head_ch,
                       value_head_ch, value_hidden=256):
    """2 x multiply-accumulates of the convolutions and linear layers of one
    forward of one position (BatchNorm, activations and softmax not counted)."""
    S2 = board_size * board_size
    f = 2 * S2 * 9 * input_channels * filters
    f += blocks * 2 * (2 * S2 * 9 * filters * filters)
    f += 2 * S2 * filters * policy_head_ch + 2 * policy_head_ch * S2 * policy_size
    f += 2 * S2 * filters * value_head_ch + 2 * value_head_ch * S2 * value_hidden + 2 * value_hidden
    return f


def make_threat_positions(n, board_size=15, seed=3):
    """Gomoku boards (int8 [n, S*S]: 0 empty, 1 black, 2 white) and sides to move (uint8 [n]) with lines planted in
    them: a few scattered stones, then two to five runs of 2-4 stones of one colour along a random direction,
    some with a gap, so that open and broken threes and fours of both colours occur.  Not reachable by legal play
    in general (stone counts are arbitrary), which the window arithmetic does not care about."""
    rng = np.random.default_rng(seed)
    S = board_size
    boards = np.zeros((n, S * S), np.int8)
    for b in range(n):
        k = int(rng.integers(0, 12))
        boards[b, rng.choice(S * S, k, replace=False)] = rng.integers(1, 3, k)
        for _ in range(int(rng.integers(2, 6))):
            colour = int(rng.integers(1, 3))
            dr, dc = [(0, 1), (1, 0), (1, 1), (1, -1)][int(rng.integers(0, 4))]
            length = int(rng.integers(2, 5))
            gap = int(rng.integers(0, length + 1)) if rng.random() < 0.4 else -1
            span = length + (gap >= 0)
            r0 = int(rng.integers(0, S - (span - 1) * dr))
            c0 = int(rng.integers((span - 1) if dc < 0 else 0, S - (span - 1) * max(dc, 0)))
            j = 0
            for i in range(span):
                if i == gap:
                    continue
                boards[b, (r0 + i * dr) * S + c0 + i * dc] = colour
                j += 1
    to_move = rng.integers(1, 3, n).astype(np.uint8)
    return boards, to_move
