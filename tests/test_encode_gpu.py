"""Encoder parity: the bf16 board tensor decodes to exactly the planes of the
CPU oracle / the reference's GomokuState (values are 0/1, so bf16 is exact)."""
import numpy as np
import pytest

from omoknuni_small_b200 import synth
from test_oracle import load_chess_golden, load_encode_golden, load_go_golden

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api(lib):
    from omoknuni_small_b200 import capi
    return capi


def run_encode(api, hist, nh, tm, S, planes, out_channels=64, dtype=0):
    import torch
    bt = api.encode_gomoku(torch.from_numpy(hist).cuda(), torch.from_numpy(nh).cuda(), torch.from_numpy(tm).cuda(), S,
                           planes, out_channels, dtype)
    torch.cuda.synchronize()
    return api.board_tensor_to_planes(bt.cpu().numpy().view(np.uint16), S, hist.shape[0], out_channels, dtype)


@pytest.mark.parametrize("planes", [17, 19])
def test_encode_matches_reference_golden(api, planes):
    games, hist, nh, tm, ref, _ = load_encode_golden()
    got, pad_zero = run_encode(api, hist, nh, tm, 15, planes)
    assert pad_zero
    assert np.array_equal(got[:, :planes], ref[:, :planes])
    assert not got[:, planes:].any()


@pytest.mark.parametrize("B,S,seed", [(1, 15, 1), (257, 15, 2), (1024, 15, 3), (40, 9, 4), (7, 19, 5)])
def test_encode_matches_oracle(api, oracle, B, S, seed):
    games, hist, nh, tm = synth.make_gomoku_games(B, S, seed=seed)
    got, pad_zero = run_encode(api, hist, nh, tm, S, 19)
    assert pad_zero and np.array_equal(got[:, :19], oracle.gomoku_encode(hist, nh, tm, S, 19))


@pytest.mark.parametrize("B,S", [(257, 15), (7, 19), (3, 31)])
def test_encode_f16_storage(api, oracle, B, S):
    """The same planes as an fp16 board tensor (both encoder kernels: the board-per-CTA one and,
    for 31x31, the per-position one)."""
    games, hist, nh, tm = synth.make_gomoku_games(B, S, seed=B)
    got, pad_zero = run_encode(api, hist, nh, tm, S, 19, dtype=api.DTYPE_F16)
    assert pad_zero and np.array_equal(got[:, :19], oracle.gomoku_encode(hist, nh, tm, S, 19))


def test_encode_edge_cases(api, oracle):
    # empty history, full 16-move history, history entries beyond n_hist are ignored
    hist = np.full((3, 16), -1, np.int16)
    hist[1] = np.arange(16) * 14
    hist[2] = np.arange(16) + 100
    nh = np.array([0, 16, 5], np.uint8)
    tm = np.array([1, 1, 2], np.uint8)
    got, pad_zero = run_encode(api, hist, nh, tm, 15, 19)
    assert pad_zero and np.array_equal(got[:, :19], oracle.gomoku_encode(hist, nh, tm, 15, 19))
    assert got[0, 16].all() and not got[0, :16].any() and not got[2, 16].any()


def test_planes_to_board_tensor_round_trip(api):
    import torch
    x = synth.make_stone_planes(33, 15, 17, seed=6)
    x[:, 3] *= 0.37                                           # a non-binary plane: must match host rounding to bf16
    bt = api.planes_to_board_tensor(torch.from_numpy(x).cuda(), 64)
    torch.cuda.synchronize()
    got = bt.cpu().numpy().view(np.uint16)
    assert np.array_equal(got, api.planes_to_board_tensor_host(x, 64))
    bt = api.planes_to_board_tensor(torch.from_numpy(x).cuda(), 64, api.DTYPE_F16)
    torch.cuda.synchronize()
    assert np.array_equal(bt.cpu().numpy().view(np.uint16), api.planes_to_board_tensor_host(x, 64, api.DTYPE_F16))


def bf16_round(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def pack_legal(legal):
    """[B,S,S] 0/1 -> int32 words, bit p of a board = cell p (little-endian bit order)."""
    B = legal.shape[0]
    flat = legal.reshape(B, -1).astype(np.uint8)
    words = (flat.shape[1] + 31) // 32
    padded = np.zeros((B, words * 32), np.uint8)
    padded[:, :flat.shape[1]] = flat
    return np.packbits(padded, axis=1, bitorder="little").view(np.uint32).astype(np.uint32).view(np.int32).reshape(B, words)


def run_encode_go(api, stones, ko, tm, legal, out_channels=64):
    import torch
    B, S = stones.shape[0], stones.shape[1]
    bt = api.encode_go(torch.from_numpy(np.ascontiguousarray(stones.reshape(B, -1), np.int8)).cuda(),
                       torch.from_numpy(np.ascontiguousarray(ko, np.int32)).cuda(),
                       torch.from_numpy(np.ascontiguousarray(tm, np.uint8)).cuda(),
                       torch.from_numpy(pack_legal(legal)).cuda(), S, out_channels)
    torch.cuda.synchronize()
    return api.board_tensor_to_planes(bt.cpu().numpy().view(np.uint16), S, B, out_channels)


@pytest.mark.parametrize("tag", ["s9", "s19"])
def test_encode_go_matches_reference_golden(api, tag):
    """The reference's GoState planes, rounded to bf16 (liberty fractions and edge distances are not
    bf16-exact; stones, colour, ko are)."""
    stones, ko, tm, legal, planes = load_go_golden(tag)
    got, pad_zero = run_encode_go(api, stones, ko, tm, legal)
    assert pad_zero
    assert np.array_equal(got[:, :10], bf16_round(planes))
    assert not got[:, 10:].any()


@pytest.mark.parametrize("B,S,fill,seed", [(300, 19, 0.45, 1), (64, 19, 0.9, 2), (50, 13, 0.6, 3), (200, 9, 0.7, 4),
                                           (3, 19, 0.0, 5), (2, 5, 1.0, 6), (5, 30, 0.5, 7)])
def test_encode_go_matches_oracle(api, oracle, B, S, fill, seed):
    """Random boards (not necessarily reachable: long chains, one-cell eyes, full and empty boards)
    with random legal subsets of the empty cells, against the C restatement."""
    rng = np.random.default_rng(seed)
    stones = (rng.random((B, S, S)) < fill) * rng.integers(1, 3, (B, S, S))
    stones = stones.astype(np.int8)
    stones[0, :, S // 2] = 1                                  # a chain across the whole board
    legal = ((stones == 0) & (rng.random((B, S, S)) < 0.8)).astype(np.uint8)
    empty = [np.flatnonzero(stones[b].reshape(-1) == 0) for b in range(B)]
    ko = np.array([int(rng.choice(e)) if len(e) and rng.random() < 0.3 else -1 for e in empty], np.int32)
    tm = rng.integers(1, 3, B).astype(np.uint8)
    got, pad_zero = run_encode_go(api, stones, ko, tm, legal, 16 if S == 30 else 64)
    want = oracle.go_encode(stones, ko, tm, legal)
    assert pad_zero and np.array_equal(got[:, :10], bf16_round(want))


def run_encode_chess(api, pieces, meta, legal_to, out_channels=64):
    import torch
    B = pieces.shape[0]
    bt = api.encode_chess(torch.from_numpy(np.ascontiguousarray(pieces, np.int8)).cuda(),
                          torch.from_numpy(np.ascontiguousarray(meta, np.int32)).cuda(),
                          torch.from_numpy(np.ascontiguousarray(legal_to, np.uint32).view(np.int32)).cuda(), out_channels)
    torch.cuda.synchronize()
    return api.board_tensor_to_planes(bt.cpu().numpy().view(np.uint16), 8, B, out_channels)


def test_encode_chess_matches_reference_golden(api):
    pieces, meta, legal_to, planes = load_chess_golden()
    got, pad_zero = run_encode_chess(api, pieces, meta, legal_to, 128)
    assert pad_zero
    assert np.array_equal(got[:, :20], bf16_round(planes))
    assert not got[:, 20:].any()


@pytest.mark.parametrize("B,C,seed", [(1, 24, 1), (700, 128, 2), (4096, 64, 3)])
def test_encode_chess_matches_oracle(api, oracle, B, C, seed):
    """Random boards and state words (not necessarily reachable: clocks beyond 100, up to 5
    occurrences, chess960, any en passant square, random destination sets)."""
    rng = np.random.default_rng(seed)
    pieces = ((rng.random((B, 64)) < 0.4) * (rng.integers(1, 7, (B, 64)) + 8 * rng.integers(0, 2, (B, 64)))).astype(np.int8)
    meta = np.stack([rng.integers(1, 3, B), rng.integers(0, 16, B), rng.integers(-1, 64, B), rng.integers(0, 160, B),
                     rng.integers(0, 2, B), rng.integers(0, 6, B)], axis=1).astype(np.int32)
    legal_to = rng.integers(0, 1 << 32, (B, 2), dtype=np.uint64).astype(np.uint32)
    got, pad_zero = run_encode_chess(api, pieces, meta, legal_to, C)
    assert pad_zero and np.array_equal(got[:, :20], bf16_round(oracle.chess_encode(pieces, meta, legal_to)))


@pytest.mark.parametrize("B,S,C", [(257, 15, 64), (3, 9, 8), (40, 19, 128)])
def test_encode_gomoku3_matches_oracle(api, oracle, B, S, C):
    """The 3-plane representation (side to move / opponent / colour) from board arrays."""
    import torch
    games, _, _, _ = synth.make_gomoku_games(B, S, seed=B, max_moves=S * S // 2)
    boards = [oracle.stones_from_moves(g, S) for g in games]
    stones = np.stack([b[0] for b in boards]); tm = np.array([b[1] for b in boards], np.uint8)
    bt = api.encode_gomoku3(torch.from_numpy(stones.reshape(B, -1)).cuda(), torch.from_numpy(tm).cuda(), S, C)
    torch.cuda.synchronize()
    got, pad_zero = api.board_tensor_to_planes(bt.cpu().numpy().view(np.uint16), S, B, C)
    assert pad_zero and np.array_equal(got[:, :3], oracle.gomoku_planes3(stones, tm)) and not got[:, 3:].any()


def test_attack_defense_matches_reference_golden(api):
    """GomokuAttackDefenseModule::compute_bonuses, stone placed, on boards with planted threes and fours
    (tests/golden/make_golden.py): the device operator gives the reference's numbers exactly."""
    import torch
    from test_oracle import load_attack_defense_golden
    for S, boards, tm, att, dfn in load_attack_defense_golden():
        a, d = api.gomoku_attack_defense(torch.from_numpy(boards).cuda(), torch.from_numpy(tm).cuda(), S, stone_placed=True)
        assert np.array_equal(a.cpu().numpy(), att) and np.array_equal(d.cpu().numpy(), dfn)
        assert np.count_nonzero(att) > 50 and np.count_nonzero(dfn) > 5


@pytest.mark.parametrize("B,S,seed", [(256, 15, 1), (33, 9, 2), (8, 19, 3), (5, 6, 4)])
def test_attack_defense_matches_oracle(api, oracle, B, S, seed):
    """Both call patterns against the CPU restatement (full recounts of every window, as the reference does it):
    the position itself - what compute_planes hands over, every plane zero, which is what the encoders write into
    planes 17 / 18 - and the position with the mover's stone on the cell."""
    import torch
    boards, tm = synth.make_threat_positions(B, S, seed=seed)
    for placed in (False, True):
        a, d = api.gomoku_attack_defense(torch.from_numpy(boards).cuda(), torch.from_numpy(tm).cuda(), S, stone_placed=placed)
        ra, rd = oracle.gomoku_attack_defense(boards, tm, S, placed)
        assert np.array_equal(a.cpu().numpy(), ra) and np.array_equal(d.cpu().numpy(), rd)
        if not placed:
            assert not ra.any() and not rd.any()
    if S == 15:
        # the encoder's planes 17 / 18 for played games are that all-zero result
        games, hist, nh, t2 = synth.make_gomoku_games(64, 15, seed=seed, max_moves=60)
        got, _ = run_encode(api, hist, nh, t2, 15, 19)
        assert not got[:, 17:19].any()
