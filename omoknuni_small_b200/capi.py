"""ctypes bindings of libomoknuni_b200.so — the Python host-side mirror of the
C ABI in include/omoknuni_b200.h.  Used by the tests and by bench.py.

Loading fails loudly when the library has not been built; there is no
fallback implementation.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libomoknuni_b200.so")

OUT_PROBS, OUT_LOGITS = 0, 1
GUARD = 32
RULES_FREESTYLE, RULES_OMOK, RULES_RENJU = 0, 1, 2
DTYPE_BF16, DTYPE_F16 = 0, 1     # storage type of board tensors and packed tower weights


class Error(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"omoknuni_b200 error {code}: {text}")
        self.code = code


class TreeView(C.Structure):
    _fields_ = [("N", C.c_void_p), ("W", C.c_void_p), ("P", C.c_void_p), ("VL", C.c_void_p),
                ("legal_bits", C.c_void_p), ("node_visits", C.c_void_p), ("child_node", C.c_void_p),
                ("n_nodes", C.c_int32), ("n_children", C.c_int32), ("pitch", C.c_int32), ("mask_words", C.c_int32)]


POLICY_FC, POLICY_CONV_PLANES = 0, 1


class NetConfig(C.Structure):
    _fields_ = [(k, C.c_int32) for k in ("board_size", "input_channels", "filters", "blocks", "policy_size",
                                          "policy_head_ch", "value_head_ch", "value_hidden", "max_batch", "device",
                                          "policy_kind", "tower_dtype")]


def widening_seed(seed, runs_before):
    """The 64-bit value that, with a node's id and a move, ranks the moves of a node under progressive widening
    during the (runs_before + 1)-th ob200_search_run of a handle created with `seed`."""
    m = (1 << 64) - 1
    z = (seed + 0x632BE59BD9B4E019 * (runs_before + 1)) & m
    z ^= z >> 31
    z = (z * 0xD6E8FEB86659FD93) & m
    z ^= z >> 32
    return z


class SearchConfig(C.Structure):
    _fields_ = [("n_trees", C.c_int32), ("sims_per_move", C.c_int32), ("leaf_batch", C.c_int32), ("max_depth", C.c_int32),
                ("c_puct", C.c_float), ("virtual_loss", C.c_int32), ("dirichlet_alpha", C.c_float),
                ("dirichlet_epsilon", C.c_float), ("value_sign", C.c_int32), ("use_transposition_table", C.c_int32),
                ("seed", C.c_uint64), ("max_children", C.c_int32), ("use_progressive_widening", C.c_int32),
                ("progressive_widening_c", C.c_float), ("progressive_widening_k", C.c_float), ("rules", C.c_int32)]


class SearchStats(C.Structure):
    _fields_ = [("simulations", C.c_int64), ("evaluations", C.c_int64), ("nodes", C.c_int64),
                ("terminal_leaves", C.c_int64), ("device_ms", C.c_double), ("wall_ms", C.c_double)]


class Counters(C.Structure):
    _fields_ = [(k, C.c_uint64) for k in ("evals", "batches", "selections", "backups", "kernel_launches")]


# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "ob200_last_error": (C.c_char_p, []),
    "ob200_version": (C.c_int, []),
    "ob200_device_count": (C.c_int, []),
    "ob200_tree_pitch": (C.c_int32, [C.c_int32]),
    "ob200_tree_mask_words": (C.c_int32, [C.c_int32]),
    "ob200_launch_puct_select": (C.c_int, [C.POINTER(TreeView), C.c_void_p, C.c_int32, C.c_float, C.c_int32, C.c_int32,
                                           C.c_void_p, C.c_void_p]),
    "ob200_launch_vl_apply": (C.c_int, [C.POINTER(TreeView), C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "ob200_launch_vl_revert": (C.c_int, [C.POINTER(TreeView), C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "ob200_launch_backup": (C.c_int, [C.POINTER(TreeView), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                      C.c_int32, C.c_void_p]),
    "ob200_launch_set_priors": (C.c_int, [C.POINTER(TreeView), C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p,
                                          C.c_void_p]),
    "ob200_launch_traverse": (C.c_int, [C.POINTER(TreeView), C.c_void_p, C.c_int32, C.c_int32, C.c_float, C.c_int32,
                                        C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ob200_tree_create": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "ob200_tree_destroy": (None, [C.c_void_p]),
    "ob200_tree_view_of": (C.c_int, [C.c_void_p, C.POINTER(TreeView)]),
    "ob200_tree_node_count": (C.c_int32, [C.c_void_p]),
    "ob200_tree_clear": (C.c_int, [C.c_void_p]),
    "ob200_tree_add_nodes": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]),
    "ob200_tree_link": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ob200_tree_select": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_float, C.c_int32, C.c_int32, C.c_void_p]),
    "ob200_tree_virtual_loss": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32]),
    "ob200_tree_backup": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32]),
    "ob200_tree_set_priors": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32]),
    "ob200_tree_read": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "ob200_tree_write": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "ob200_board_tensor_positions": (C.c_int64, [C.c_int32, C.c_int32]),
    "ob200_board_tensor_bytes": (C.c_int64, [C.c_int32, C.c_int32, C.c_int32]),
    "ob200_launch_encode_gomoku": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                             C.c_int32, C.c_void_p, C.c_void_p]),
    "ob200_launch_encode_gomoku_dt": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                                C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "ob200_launch_encode_go": (C.c_int, [C.c_void_p] * 4 + [C.c_int32] * 3 + [C.c_void_p, C.c_void_p]),
    "ob200_launch_encode_gomoku3": (C.c_int, [C.c_void_p, C.c_void_p] + [C.c_int32] * 3 + [C.c_void_p, C.c_void_p]),
    "ob200_launch_gomoku_attack_defense": (C.c_int, [C.c_void_p, C.c_void_p] + [C.c_int32] * 3 + [C.c_void_p] * 3),
    "ob200_launch_encode_chess": (C.c_int, [C.c_void_p] * 3 + [C.c_int32] * 2 + [C.c_void_p, C.c_void_p]),
    "ob200_launch_planes_to_board_tensor": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                                      C.c_void_p]),
    "ob200_launch_planes_to_board_tensor_dt": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                         C.c_void_p, C.c_void_p]),
    "ob200_launch_conv3x3_dt": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                          C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "ob200_pack_conv3x3_weights_dt": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                C.c_void_p]),
    "ob200_launch_conv3x3": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                       C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "ob200_packed_conv3x3_bytes": (C.c_int64, [C.c_int32, C.c_int32]),
    "ob200_pack_conv3x3_weights": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "ob200_net_create": (C.c_int, [C.POINTER(NetConfig), C.POINTER(C.c_void_p)]),
    "ob200_net_destroy": (None, [C.c_void_p]),
    "ob200_net_set_tensor": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int64]),
    "ob200_net_finalize": (C.c_int, [C.c_void_p]),
    "ob200_net_infer_planes": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32]),
    "ob200_net_infer_gomoku": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                         C.c_void_p, C.c_int32]),
    "ob200_net_submit_gomoku": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                          C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]),
    "ob200_net_wait": (C.c_int, [C.c_void_p, C.c_int32]),
    "ob200_net_forward_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32,
                                           C.c_void_p]),
    "ob200_net_forward_gomoku_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                                  C.c_void_p, C.c_int32, C.c_void_p]),
    "ob200_debug_bounded_wait": (C.c_int, [C.c_int32, C.c_void_p]),
    "ob200_net_debug_tower_output": (C.c_void_p, [C.c_void_p]),
    "ob200_net_debug_tower_path": (C.c_int32, [C.c_void_p]),
    "ob200_net_tower_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "ob200_net_input_tensor_channels": (C.c_int32, [C.c_void_p]),
    "ob200_net_value_head_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "ob200_value_head_noalloc_capacity": (C.c_int64, []),
    "ob200_device_error_code": (C.c_int, [C.POINTER(C.c_int32)]),
    "ob200_search_create": (C.c_int, [C.c_void_p, C.POINTER(SearchConfig), C.POINTER(C.c_void_p)]),
    "ob200_search_destroy": (None, [C.c_void_p]),
    "ob200_search_run": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_float, C.c_void_p, C.c_void_p,
                                   C.POINTER(SearchStats)]),
    "ob200_search_debug_tree": (C.c_int, [C.c_void_p, C.POINTER(TreeView), C.POINTER(C.c_int32)]),
    "ob200_search_debug_hooks": (C.c_int, [C.c_void_p, C.c_float, C.c_int32]),
    "ob200_search_debug_phases": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "ob200_search_debug_record": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "ob200_copy_to_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64]),
    "ob200_get_counters": (C.c_int, [C.POINTER(Counters)]),
    "ob200_reset_counters": (None, []),
}

_lib = None


def lib():
    """The loaded library.  Raises when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise Error(-1, f"{LIB_PATH} is missing: run `python -m omoknuni_small_b200.build` (there is no fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        raise Error(rc, lib().ob200_last_error().decode())


def counters():
    c = Counters()
    check(lib().ob200_get_counters(C.byref(c)))
    return {k: getattr(c, k) for k, _ in Counters._fields_}


def device_error_code():
    v = C.c_int32(0)
    check(lib().ob200_device_error_code(C.byref(v)))
    return v.value


def _ptr(t):
    """Device pointer of a torch tensor (or None)."""
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class DeviceTree:
    """Edge statistics on the device (torch tensors own the memory) + the view
    struct the launchers take.  `tree` is a dict as synth.make_selection_tree
    returns; an optional 'child_node' [n_nodes, pitch] int32 enables descent."""

    def __init__(self, tree, device="cuda:0"):
        import torch
        self.torch = torch
        self.n_nodes, self.pitch = tree["N"].shape
        self.n_children = int(tree["n_children"])
        self.t = {k: torch.from_numpy(np.ascontiguousarray(tree[k])).to(device)
                  for k in ("N", "W", "P", "VL", "node_visits") if k in tree}
        self.t["legal_bits"] = torch.from_numpy(np.ascontiguousarray(tree["legal_bits"]).view(np.int32)).to(device)
        if tree.get("child_node") is not None:
            self.t["child_node"] = torch.from_numpy(np.ascontiguousarray(tree["child_node"])).to(device)
        self.mask_words = tree["legal_bits"].shape[1]
        self.device = device
        self.view = TreeView(self.t["N"].data_ptr(), self.t["W"].data_ptr(), self.t["P"].data_ptr(),
                             self.t["VL"].data_ptr(), self.t["legal_bits"].data_ptr(),
                             self.t["node_visits"].data_ptr(),
                             self.t["child_node"].data_ptr() if "child_node" in self.t else None,
                             self.n_nodes, self.n_children, self.pitch, self.mask_words)

    def host(self, key):
        return self.t[key].cpu().numpy()

    def select(self, node_ids=None, c_puct=1.5, vl_value=3, apply_vl=True, out=None):
        torch = self.torch
        n = self.n_nodes if node_ids is None else node_ids.numel()
        if out is None:
            out = torch.empty(n, dtype=torch.int32, device=self.device)
        check(lib().ob200_launch_puct_select(C.byref(self.view), _ptr(node_ids), n, c_puct, vl_value, int(apply_vl),
                                             _ptr(out), _stream()))
        return out

    def vl_apply(self, sel, vl_value=3, node_ids=None):
        check(lib().ob200_launch_vl_apply(C.byref(self.view), _ptr(node_ids), _ptr(sel), sel.numel(), vl_value, _stream()))

    def vl_revert(self, sel, vl_value=3, node_ids=None):
        check(lib().ob200_launch_vl_revert(C.byref(self.view), _ptr(node_ids), _ptr(sel), sel.numel(), vl_value, _stream()))

    def backup(self, paths, path_len, leaf_values, vl_value=3):
        n, max_depth, _ = paths.shape
        check(lib().ob200_launch_backup(C.byref(self.view), _ptr(paths), _ptr(path_len), _ptr(leaf_values), n, max_depth,
                                        vl_value, _stream()))

    def set_priors(self, node_ids, policy, slot_action=None):
        check(lib().ob200_launch_set_priors(C.byref(self.view), _ptr(node_ids), policy.shape[0], _ptr(policy),
                                            policy.shape[1], _ptr(slot_action), _stream()))

    def traverse(self, roots, sims_per_tree, c_puct=1.5, vl_value=3, max_depth=64):
        torch = self.torch
        n = roots.numel() * sims_per_tree
        paths = torch.zeros((n, max_depth, 2), dtype=torch.int32, device=self.device)
        plen = torch.zeros(n, dtype=torch.int32, device=self.device)
        check(lib().ob200_launch_traverse(C.byref(self.view), _ptr(roots), roots.numel(), sims_per_tree, c_puct, vl_value,
                                          max_depth, _ptr(paths), _ptr(plen), _stream()))
        return paths, plen


# ---- board tensors -------------------------------------------------------------
def board_positions(board_size, B):
    return int(lib().ob200_board_tensor_positions(board_size, B))


def board_tensor_to_planes(bt_u16, board_size, B, channels, dtype=DTYPE_BF16):
    """16-bit NHWC board tensor (numpy uint16 view, flat, `channels` rounded up to 8
    per position) -> fp32 planes [B, channels, S, S] plus a flag telling whether
    every padding / guard element is zero.  Host-side helper for tests."""
    S, GP = board_size, board_size + 1
    slots = GP * GP
    PT = board_positions(S, B)
    Cp = (channels + 7) // 8 * 8
    a = np.asarray(bt_u16).reshape(-1)[: PT * Cp].reshape(PT, Cp)
    f = a.view(np.float16).astype(np.float32) if dtype == DTYPE_F16 else (a.astype(np.uint32) << 16).view(np.float32)
    body = f[GUARD:GUARD + B * slots].reshape(B, GP, GP, Cp)
    planes = body[:, :S, :S, :channels].transpose(0, 3, 1, 2)
    pad_zero = (not f[:GUARD].any() and not f[GUARD + B * slots:].any()
                and not body[:, S, :, :].any() and not body[:, :, S, :].any())
    return np.ascontiguousarray(planes), bool(pad_zero)


def planes_to_board_tensor_host(planes, out_channels, dtype=DTYPE_BF16):
    """fp32 planes [B, C, S, S] -> 16-bit NHWC board tensor as a flat numpy uint16
    array (round to nearest even), the host-side twin of the device conversion."""
    B, Cc, S, _ = planes.shape
    GP = S + 1
    PT = board_positions(S, B)
    full = np.zeros((B, GP, GP, out_channels), np.float32)
    full[:, :S, :S, :Cc] = planes.transpose(0, 2, 3, 1)
    u = full.view(np.uint32)
    r = full.astype(np.float16).view(np.uint16) if dtype == DTYPE_F16 else ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    out = np.zeros((PT, out_channels), np.uint16)
    out[GUARD:GUARD + B * GP * GP] = r.reshape(B * GP * GP, out_channels)
    return out.reshape(-1)


def encode_gomoku(history, n_hist, to_move, board_size=15, planes=19, out_channels=64, dtype=DTYPE_BF16, out=None):
    """Device tensors in (int16 [B,16], uint8 [B], uint8 [B]) -> board tensor
    (torch int16 tensor holding the bf16 / fp16 bits; `out`: a tensor of that size to write into)."""
    import torch
    B = history.shape[0]
    nbytes = int(lib().ob200_board_tensor_bytes(board_size, B, out_channels))
    if out is None:
        out = torch.empty(nbytes // 2, dtype=torch.int16, device=history.device)
    assert out.numel() * out.element_size() == nbytes
    check(lib().ob200_launch_encode_gomoku_dt(_ptr(history), _ptr(n_hist), _ptr(to_move), B, board_size, planes,
                                              out_channels, dtype, _ptr(out), _stream()))
    return out


def encode_go(stones, ko_point, to_move, legal_bits, board_size, out_channels=64):
    """Device tensors in (int8 [B,S*S], int32 [B], uint8 [B], int32 [B,ceil(S*S/32)] bit masks)
    -> bf16 board tensor (int16 view) with the reference's 10 Go planes."""
    import torch
    B = stones.shape[0]
    nbytes = int(lib().ob200_board_tensor_bytes(board_size, B, out_channels))
    out = torch.empty(nbytes // 2, dtype=torch.int16, device=stones.device)
    check(lib().ob200_launch_encode_go(_ptr(stones), _ptr(ko_point), _ptr(to_move), _ptr(legal_bits), B, board_size,
                                       out_channels, _ptr(out), _stream()))
    return out


def encode_gomoku3(stones, to_move, board_size, out_channels=64):
    """Device tensors in (int8 [B,S*S], uint8 [B]) -> bf16 board tensor with the 3-plane representation."""
    import torch
    B = stones.shape[0]
    nbytes = int(lib().ob200_board_tensor_bytes(board_size, B, out_channels))
    out = torch.empty(nbytes // 2, dtype=torch.int16, device=stones.device)
    check(lib().ob200_launch_encode_gomoku3(_ptr(stones), _ptr(to_move), B, board_size, out_channels, _ptr(out), _stream()))
    return out


def gomoku_attack_defense(stones, to_move, board_size, stone_placed=False):
    """Device tensors in (int8 [B,S*S], uint8 [B]) -> (attack, defense) fp32 [B,S*S] each."""
    import torch
    B = stones.shape[0]
    att = torch.empty((B, board_size * board_size), dtype=torch.float32, device=stones.device)
    dfn = torch.empty_like(att)
    check(lib().ob200_launch_gomoku_attack_defense(_ptr(stones), _ptr(to_move), B, board_size, int(stone_placed), _ptr(att),
                                                   _ptr(dfn), _stream()))
    return att, dfn


def encode_chess(pieces, meta, legal_to, out_channels=64):
    """Device tensors in (int8 [B,64], int32 [B,6], int32 [B,2] bit masks) -> bf16 board tensor
    (int16 view, board_size 8) with the reference's 20 chess planes."""
    import torch
    B = pieces.shape[0]
    nbytes = int(lib().ob200_board_tensor_bytes(8, B, out_channels))
    out = torch.empty(nbytes // 2, dtype=torch.int16, device=pieces.device)
    check(lib().ob200_launch_encode_chess(_ptr(pieces), _ptr(meta), _ptr(legal_to), B, out_channels, _ptr(out), _stream()))
    return out


def planes_to_board_tensor(planes, out_channels, dtype=DTYPE_BF16):
    import torch
    B, Cc, S, _ = planes.shape
    nbytes = int(lib().ob200_board_tensor_bytes(S, B, out_channels))
    out = torch.empty(nbytes // 2, dtype=torch.int16, device=planes.device)
    check(lib().ob200_launch_planes_to_board_tensor_dt(_ptr(planes), B, Cc, S, out_channels, dtype, _ptr(out), _stream()))
    return out


def pack_conv3x3(w_oihw, scale, cin=64, dtype=DTYPE_BF16):
    """fp32 [cout, cin_real, 3, 3] (+ per-output-channel scale or None) -> packed
    bf16 / fp16 image as numpy uint16."""
    w = np.ascontiguousarray(w_oihw, np.float32)
    cout, cin_real = w.shape[:2]
    out = np.empty(int(lib().ob200_packed_conv3x3_bytes(cin, cout)) // 2, np.uint16)
    sc = None if scale is None else np.ascontiguousarray(scale, np.float32)
    check(lib().ob200_pack_conv3x3_weights_dt(w.ctypes.data_as(C.c_void_p), None if sc is None else sc.ctypes.data_as(C.c_void_p),
                                              cout, cin_real, cin, dtype, out.ctypes.data_as(C.c_void_p)))
    return out


def conv3x3(x_bt, packed_w, bias, residual_bt, B, board_size, cin=64, cout=64, relu=True, out=None, dtype=DTYPE_BF16):
    """One conv layer on device board tensors (torch int16 tensors with bf16 / fp16 bits)."""
    import torch
    if out is None:
        nbytes = int(lib().ob200_board_tensor_bytes(board_size, B, cout))
        out = torch.zeros(nbytes // 2, dtype=torch.int16, device=x_bt.device)
    check(lib().ob200_launch_conv3x3_dt(_ptr(x_bt), _ptr(packed_w), _ptr(bias), _ptr(residual_bt), _ptr(out), B, board_size,
                                        cin, cout, int(relu), dtype, _stream()))
    return out


# ---- network handle ------------------------------------------------------------
class Net:
    """The residual policy/value network on one GPU (host-side mirror of the
    reference's ResNetModel: constructor arguments in the same order, weights
    under the same names, inference on host buffers)."""

    def __init__(self, input_channels, board_size, blocks, filters, policy_size, policy_head_ch=32, value_head_ch=32,
                 value_hidden=256, max_batch=1024, device=0, policy_kind=POLICY_FC, tower_dtype=DTYPE_BF16):
        self.cfg = NetConfig(board_size, input_channels, filters, blocks, policy_size or board_size * board_size,
                             policy_head_ch, value_head_ch, value_hidden, max_batch, device, policy_kind, tower_dtype)
        self.tower_dtype = tower_dtype
        self.h = C.c_void_p()
        check(lib().ob200_net_create(C.byref(self.cfg), C.byref(self.h)))
        self.policy_size = self.cfg.policy_size
        self.board_size = board_size

    def load(self, weights):
        """weights: dict name -> numpy array under the reference's parameter names."""
        for name, arr in weights.items():
            a = np.ascontiguousarray(arr, np.float32)
            check(lib().ob200_net_set_tensor(self.h, name.encode(), a.ctypes.data_as(C.c_void_p), a.size))
        check(lib().ob200_net_finalize(self.h))
        return self

    def infer_planes(self, planes, out_kind=OUT_PROBS):
        x = np.ascontiguousarray(planes, np.float32)
        B, Cc = x.shape[:2]
        pol = np.empty((B, self.policy_size), np.float32)
        val = np.empty(B, np.float32)
        check(lib().ob200_net_infer_planes(self.h, x.ctypes.data_as(C.c_void_p), B, Cc, pol.ctypes.data_as(C.c_void_p),
                                           val.ctypes.data_as(C.c_void_p), out_kind))
        return pol, val

    def infer_gomoku(self, history, n_hist, to_move, out_kind=OUT_PROBS, out=None):
        """out: optional (policy [B, A] float32, value [B] float32) numpy arrays to fill; arrays in
        page-locked memory are written by the copy engine directly."""
        h = np.ascontiguousarray(history, np.int16)
        nh = np.ascontiguousarray(n_hist, np.uint8)
        tm = np.ascontiguousarray(to_move, np.uint8)
        B = h.shape[0]
        if out is not None:
            pol, val = out
            assert pol.dtype == np.float32 and val.dtype == np.float32 and pol.flags.c_contiguous and val.flags.c_contiguous
            assert pol.shape == (B, self.policy_size) and val.shape == (B,)
        else:
            pol = np.empty((B, self.policy_size), np.float32)
            val = np.empty(B, np.float32)
        check(lib().ob200_net_infer_gomoku(self.h, h.ctypes.data_as(C.c_void_p), nh.ctypes.data_as(C.c_void_p),
                                           tm.ctypes.data_as(C.c_void_p), B, pol.ctypes.data_as(C.c_void_p),
                                           val.ctypes.data_as(C.c_void_p), out_kind))
        return pol, val

    def submit_gomoku(self, history, n_hist, to_move, out, out_kind=OUT_PROBS):
        """Asynchronous infer_gomoku: enqueues the call and returns a ticket for wait().  The arrays (C-contiguous
        int16 / uint8 / uint8 inputs, float32 outputs in `out`) must stay alive and untouched until then; at most two
        calls may be pending."""
        pol, val = out
        B = history.shape[0]
        assert history.dtype == np.int16 and n_hist.dtype == np.uint8 and to_move.dtype == np.uint8
        assert pol.dtype == np.float32 and val.dtype == np.float32 and pol.shape == (B, self.policy_size) and val.shape == (B,)
        ticket = C.c_int32(-1)
        check(lib().ob200_net_submit_gomoku(self.h, history.ctypes.data_as(C.c_void_p), n_hist.ctypes.data_as(C.c_void_p),
                                            to_move.ctypes.data_as(C.c_void_p), B, pol.ctypes.data_as(C.c_void_p),
                                            val.ctypes.data_as(C.c_void_p), out_kind, C.byref(ticket)))
        return ticket.value

    def wait(self, ticket):
        check(lib().ob200_net_wait(self.h, ticket))

    def input_tensor_channels(self):
        return int(lib().ob200_net_input_tensor_channels(self.h))

    def forward_device(self, input_bt, B, policy_out, value_out, out_kind=OUT_PROBS):
        check(lib().ob200_net_forward_device(self.h, _ptr(input_bt), B, _ptr(policy_out), _ptr(value_out), out_kind,
                                             _stream()))

    def forward_gomoku_device(self, history, n_hist, to_move, policy_out, value_out, out_kind=OUT_PROBS):
        """encode -> tower -> heads on device move histories (torch tensors: int16 [B,16], uint8 [B], uint8 [B])."""
        check(lib().ob200_net_forward_gomoku_device(self.h, _ptr(history), _ptr(n_hist), _ptr(to_move), history.shape[0],
                                                    _ptr(policy_out), _ptr(value_out), out_kind, _stream()))

    def tower_device(self, input_bt, B):
        """The residual tower alone on a device input tensor (asynchronous)."""
        check(lib().ob200_net_tower_device(self.h, _ptr(input_bt), B, _stream()))

    def tower_output_ptr(self):
        return lib().ob200_net_debug_tower_output(self.h)

    def tower_path(self):
        """0 launch per layer, 1 one cooperative launch, 2 boards resident in shared memory (last forward)."""
        return int(lib().ob200_net_debug_tower_path(self.h))

    def value_head_noalloc(self, tower_ptr, B, value_out):
        """Value head from a tower output already on the device, using only the
        library's built-in scratch array (no allocation anywhere)."""
        check(lib().ob200_net_value_head_noalloc(self.h, C.c_void_p(tower_ptr), B, _ptr(value_out), _stream()))

    def close(self):
        if self.h:
            lib().ob200_net_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- leaf-parallel search ---------------------------------------------------------
class Search:
    """Leaf-parallel MCTS over a group of Gomoku games on one GPU (host-side mirror of
    MCTSEngine::search for many games at once)."""

    def __init__(self, net, n_trees=64, sims_per_move=800, leaf_batch=1024, max_depth=64, c_puct=1.5, virtual_loss=3,
                 dirichlet_alpha=0.3, dirichlet_epsilon=0.25, value_sign=1, transposition_table=False, seed=0,
                 max_children=0, progressive_widening=None, rules=0):
        """progressive_widening: None (off, as the reference's shipped configuration) or (c, k) of MCTSSettings.
        rules: RULES_FREESTYLE or RULES_OMOK."""
        self.net = net                       # keep the network alive
        pw = progressive_widening
        self.cfg = SearchConfig(n_trees, sims_per_move, leaf_batch, max_depth, c_puct, virtual_loss, dirichlet_alpha,
                                dirichlet_epsilon, value_sign, int(transposition_table), seed, max_children,
                                int(pw is not None), pw[0] if pw else 0.0, pw[1] if pw else 0.0, rules)
        self.h = C.c_void_p()
        check(lib().ob200_search_create(net.h, C.byref(self.cfg), C.byref(self.h)))

    def run(self, move_lists, temperature=1.0):
        """move_lists: one sequence of actions per tree.  Returns (pi [T,225], visits [T,225], stats dict)."""
        T = self.cfg.n_trees
        assert len(move_lists) == T
        stride = max(1, max(len(m) for m in move_lists))
        moves = np.full((T, stride), -1, np.int16)
        n = np.zeros(T, np.int32)
        for t, m in enumerate(move_lists):
            moves[t, :len(m)] = m
            n[t] = len(m)
        pi = np.zeros((T, 225), np.float32)
        visits = np.zeros((T, 225), np.int32)
        st = SearchStats()
        check(lib().ob200_search_run(self.h, moves.ctypes.data_as(C.c_void_p), n.ctypes.data_as(C.c_void_p), stride,
                                     temperature, pi.ctypes.data_as(C.c_void_p), visits.ctypes.data_as(C.c_void_p),
                                     C.byref(st)))
        return pi, visits, {k: getattr(st, k) for k, _ in SearchStats._fields_}

    def debug_hooks(self, value_quantum=0.0, record_rounds=0):
        """Test hooks: round network values to multiples of 1 / value_quantum; keep the network outputs of the
        root evaluation and of the first `record_rounds` rounds of each run."""
        check(lib().ob200_search_debug_hooks(self.h, value_quantum, record_rounds))
        self._rec_rounds = record_rounds

    def phase_timing(self, enable=True):
        """Switches per-phase event timing of the following runs on or off; returns the sums (ms) of the last timed run
        as a dict: descent, leaf_positions, network, expansion, backup."""
        out = (C.c_double * 5)()
        check(lib().ob200_search_debug_phases(self.h, int(enable), out))
        return dict(zip(("descent", "leaf_positions", "network", "expansion", "backup"), [float(v) for v in out]))

    def record(self):
        """(policy [R + 1, L, 225], value [R + 1, L], noise [T, 228]) of the last run, as numpy arrays."""
        pp, vp, nz = C.c_void_p(), C.c_void_p(), C.c_void_p()
        check(lib().ob200_search_debug_record(self.h, C.byref(pp), C.byref(vp), C.byref(nz)))
        R, L, T = self._rec_rounds, self.cfg.leaf_batch, self.cfg.n_trees

        def pull(ptr, shape):
            a = np.empty(shape, np.float32)
            check(lib().ob200_copy_to_host(a.ctypes.data_as(C.c_void_p), ptr, a.nbytes))
            return a
        return pull(pp, (R + 1, L, 225)), pull(vp, (R + 1, L)), pull(nz, (T, 228))

    def tree(self):
        """Host copies of the search's tree arrays (for tests): dict of numpy arrays + nodes used."""
        v = TreeView()
        used = C.c_int32(0)
        check(lib().ob200_search_debug_tree(self.h, C.byref(v), C.byref(used)))
        n, pitch, mw = used.value, v.pitch, v.mask_words

        def pull(ptr, count, dtype):
            a = np.empty(count, dtype)
            check(lib().ob200_copy_to_host(a.ctypes.data_as(C.c_void_p), C.c_void_p(ptr), a.nbytes))
            return a
        return {"N": pull(v.N, n * pitch, np.int32).reshape(n, pitch), "W": pull(v.W, n * pitch, np.float32).reshape(n, pitch),
                "P": pull(v.P, n * pitch, np.float32).reshape(n, pitch), "VL": pull(v.VL, n * pitch, np.int32).reshape(n, pitch),
                "child_node": pull(v.child_node, n * pitch, np.int32).reshape(n, pitch),
                "legal_bits": pull(v.legal_bits, n * mw, np.uint32).reshape(n, mw),
                "node_visits": pull(v.node_visits, n, np.int32), "n_children": v.n_children, "nodes": n}

    def close(self):
        if self.h:
            lib().ob200_search_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
