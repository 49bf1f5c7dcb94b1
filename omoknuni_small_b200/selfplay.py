"""Self-play over the device search: many Gomoku games advance together, one
search call per ply for the whole group, finished games are written out and
their slot starts a new game.

Takes the place of SelfPlayManager::generateGames / generateGame (reference
src/selfplay/self_play_manager.cpp:309-473,536-890) for Gomoku: temperature
schedule (high until `temperature_threshold` moves, then low, :630-640), the
move drawn from the visit distribution, and one JSON record per game with the
reference's fields (game_type, board_size, winner, total_time_ms, game_id,
moves, policies — as in its data/self_play_games/*.json, which its trainer
reads back, alphazero_train.py:51-82).
"""
import json
import os
import time

import numpy as np

GAME_TYPE_GOMOKU = 3   # core::GameType::GOMOKU (reference include/core/igamestate.h:18-24)


def gomoku_result(moves, board_size=15, rules=0):
    """0 ongoing, 1 BLACK won, 2 WHITE won, 3 draw — judged on the last move, five
    or more in a row wins (reference src/games/gomoku/gomoku_rules.cpp:71-100); under Renju
    (rules 2) BLACK needs exactly five and no longer line through the stone
    (src/games/gomoku/gomoku_state.cpp:812-843)."""
    n = len(moves)
    if n == 0:
        return 0
    S = board_size
    board = np.zeros(S * S, np.int8)
    board[np.asarray(moves[0::2], np.int64)] = 1
    board[np.asarray(moves[1::2], np.int64)] = 2
    last = int(moves[-1])
    who = int(board[last])
    r0, c0 = divmod(last, S)
    runs = []
    for dr, dc in ((1, 0), (0, 1), (1, 1), (1, -1)):
        run = 1
        for sgn in (1, -1):
            r, c = r0 + sgn * dr, c0 + sgn * dc
            while 0 <= r < S and 0 <= c < S and board[r * S + c] == who:
                run += 1
                r += sgn * dr
                c += sgn * dc
        runs.append(run)
    won = (5 in runs and max(runs) == 5) if (rules == 2 and who == 1) else max(runs) >= 5
    if won:
        return who
    return 3 if n >= S * S else 0


def visits_to_policy(visits, temperature):
    """MCTSEngine::getActionProbabilities (reference src/mcts/mcts_engine_tree.cpp:389-465):
    (n / n_max)^(1/T) normalised; one-hot on the most visited move for T < 0.01."""
    v = np.asarray(visits, np.float64)
    pi = np.zeros_like(v)
    if v.max() <= 0:
        return pi.astype(np.float32)
    if temperature < 0.01:
        pi[int(v.argmax())] = 1.0
    else:
        pi = (v / v.max()) ** (1.0 / temperature)
        pi /= pi.sum()
    return pi.astype(np.float32)


class SelfPlay:
    def __init__(self, search, board_size=15, temperature_threshold=30, high_temperature=1.0, low_temperature=0.1,
                 max_moves=0, seed=0, out_dir=None):
        self.search, self.S = search, board_size
        self.threshold, self.high, self.low = temperature_threshold, high_temperature, low_temperature
        self.max_moves = max_moves or board_size * board_size
        self.rng = np.random.default_rng(seed)
        self.out_dir = out_dir
        if out_dir:
            os.makedirs(out_dir, exist_ok=True)

    def generate_games(self, n_games, openings=None):
        """Plays until n_games are finished; returns the list of records."""
        T = self.search.cfg.n_trees
        slots = [list(openings[i]) if openings else [] for i in range(T)]
        first_ply = [len(s) for s in slots]
        policies = [[] for _ in range(T)]
        started = [time.time()] * T
        records, next_id, stamp = [], 0, time.strftime("%Y%m%d_%H%M%S")
        while len(records) < n_games:
            _, visits, _ = self.search.run(slots, temperature=1.0)
            for t in range(T):
                ply = len(slots[t])
                temp = self.high if ply < self.threshold else self.low
                pi = visits_to_policy(visits[t], temp)
                if pi.sum() <= 0:                       # no legal move was visited: treat the game as drawn
                    result = 3
                else:
                    move = int(pi.argmax()) if temp < 0.01 else int(self.rng.choice(len(pi), p=pi / pi.sum()))
                    slots[t].append(move)
                    policies[t].append(pi.tolist())
                    result = gomoku_result(slots[t], self.S, self.search.cfg.rules)
                    if result == 0 and len(slots[t]) >= self.max_moves:
                        result = 3
                if result:
                    rec = {"game_type": GAME_TYPE_GOMOKU, "board_size": self.S, "winner": 0 if result == 3 else result,
                           "total_time_ms": int((time.time() - started[t]) * 1000), "game_id": f"{stamp}_{next_id}",
                           "moves": slots[t][first_ply[t]:] if first_ply[t] else slots[t], "policies": policies[t]}
                    if first_ply[t]:
                        rec["opening"] = slots[t][:first_ply[t]]
                    records.append(rec)
                    if self.out_dir:
                        with open(os.path.join(self.out_dir, f"game_{rec['game_id']}.json"), "w") as f:
                            json.dump(rec, f)
                    next_id += 1
                    slots[t], policies[t], first_ply[t], started[t] = [], [], 0, time.time()
        return records[:n_games]
