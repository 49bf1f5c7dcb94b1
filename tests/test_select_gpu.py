"""Parity of the selection / virtual-loss / backup / traversal kernels with the
CPU oracle, through the C ABI: bit-exact indices and integer state."""
import os

import numpy as np
import pytest

from omoknuni_small_b200 import synth

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def api(lib):
    import torch
    from omoknuni_small_b200 import capi
    torch.cuda.init()
    return capi


@pytest.mark.parametrize("n_nodes,nc,seed", [(4096, 225, 7), (257, 362, 8), (16384, 362, 12), (64, 4672, 9), (300, 3, 10), (33, 1, 11),
                                               (12288, 260, 13), (300, 1024, 14), (70, 8192, 15), (33, 1027, 16), (1500, 256, 17)])
def test_select_apply_revert_bit_exact(api, oracle, n_nodes, nc, seed):
    import torch
    t = synth.make_selection_tree(n_nodes, nc, seed=seed)
    ref = synth.copy_tree(t)
    dt = api.DeviceTree(t)
    sel = dt.select(c_puct=1.5, vl_value=3, apply_vl=True)
    sel_ref = oracle.puct_select(ref, c_puct=1.5, vl_value=3, apply_vl=True)
    torch.cuda.synchronize()
    assert np.array_equal(sel.cpu().numpy(), sel_ref)
    assert np.array_equal(dt.host("VL"), ref["VL"])
    dt.vl_revert(sel, 3)
    oracle.vl_revert(ref, sel_ref, 3)
    assert np.array_equal(dt.host("VL"), ref["VL"]) and np.array_equal(ref["VL"], t["VL"])


@pytest.mark.parametrize("tag", ["g225", "c4672", "n3"])
def test_select_matches_reference_golden(api, tag):
    g = np.load(os.path.join(GOLD, "select_golden.npz"))
    n_nodes, nc, seed = [int(v) for v in g[tag + "_shape"]]
    t = synth.make_selection_tree(n_nodes, nc, seed=seed)
    dt = api.DeviceTree(t)
    sel = dt.select(c_puct=1.5, vl_value=3, apply_vl=True).cpu().numpy()
    assert np.array_equal(sel, g[tag + "_sel"])
    rows = np.arange(n_nodes)
    assert np.array_equal(dt.host("VL")[rows, sel], g[tag + "_vl_after_apply"])


def test_select_edge_cases(api, oracle):
    import torch
    t = synth.make_selection_tree(64, 225, seed=21)
    t["legal_bits"][0] = 0                                  # node without children -> -1
    t["legal_bits"][1] = 0; t["legal_bits"][1, 7] = 1 << 0  # one child, the last slot (224)
    t["P"][2] = 0; t["N"][2] = 0; t["W"][2] = 0; t["VL"][2] = 0   # all scores equal -> lowest legal slot
    t["W"][3, :225] = np.nan                                # no score compares greater -> least visited
    t["W"][4, :225] = -np.inf
    t["node_visits"][5] = 0                                 # unvisited parent: exploration term is 0
    t["VL"][6] = 1000                                       # large virtual loss everywhere
    ref = synth.copy_tree(t)
    ids = np.array([0, 1, 2, 3, 4, 5, 6, 7, 7, 63, 1], np.int32)   # with repeats
    dt = api.DeviceTree(t)
    sel = dt.select(torch.from_numpy(ids).cuda(), c_puct=1.5, vl_value=3, apply_vl=False).cpu().numpy()
    sel_ref = oracle.puct_select(ref, ids, c_puct=1.5, vl_value=3, apply_vl=False)
    assert np.array_equal(sel, sel_ref)
    assert sel[0] == -1 and sel[1] == 224
    # empty launch is fine
    dt.select(torch.zeros(0, dtype=torch.int32, device="cuda"))


def test_select_full_size_pass(api, oracle):
    """The benchmark's full size, 65,536 nodes x 225 children: selection, virtual loss apply and
    revert equal the oracle node for node, and the pass leaves the tree as it found it."""
    import torch
    t = synth.make_selection_tree(65536, 225, seed=7)
    ref = synth.copy_tree(t)
    dt = api.DeviceTree(t)
    sel = dt.select(c_puct=1.5, vl_value=3, apply_vl=True)
    sel_ref = oracle.puct_select(ref, c_puct=1.5, vl_value=3, apply_vl=True)
    torch.cuda.synchronize()
    assert np.array_equal(sel.cpu().numpy(), sel_ref)
    assert np.array_equal(dt.host("VL"), ref["VL"])
    dt.vl_revert(sel, 3)
    assert np.array_equal(dt.host("VL"), t["VL"])
    assert api.device_error_code() == 0


def test_select_wide_rows_edge_cases(api, oracle):
    """Chess-wide rows (4,672 slots) take the segmented kernel: the same edge cases, a node
    list with repeats and out-of-range ids, more (node, segment) pairs than warps."""
    import torch
    nc = 4672
    t = synth.make_selection_tree(1500, nc, seed=31)
    t["legal_bits"][0] = 0                                  # node without children -> -1
    t["legal_bits"][1] = 0; t["legal_bits"][1, (nc - 1) >> 5] = 1 << ((nc - 1) & 31)   # one child: the last slot
    t["P"][2] = 0; t["N"][2] = 0; t["W"][2] = 0; t["VL"][2] = 0   # all scores equal -> lowest legal slot
    t["W"][3, :nc] = np.nan                                 # no score compares greater -> least visited
    t["W"][4, :nc] = -np.inf
    t["node_visits"][5] = 0                                 # unvisited parent: exploration term is 0
    t["VL"][6] = 1000                                       # large virtual loss everywhere
    t["P"][7, :nc] = 1.0 / nc; t["N"][7] = 3; t["W"][7] = 1.5; t["VL"][7] = 0   # a wide tie at a non-zero score
    t["N"][8, 100:140] = 2 ** 24 + 3; t["W"][8, 100:140] = 2.0 ** 24    # visit counts beyond the fast conversion's range
    t["N"][8, 3000] = 2 ** 30; t["W"][8, 3000] = 2.0 ** 30
    t["VL"][9, 5] = -2; t["VL"][9, 4000] = -1               # negative counts take the conversions proper as well
    t["N"][10] = 1; t["VL"][10] = 0; t["W"][10] = 0.0; t["P"][10] = 0.0   # a tie of zeros of both signs across segments:
    t["W"][10, :600] = -0.0; t["P"][10, :600] = -0.0        # -0 == +0, so the lowest existing slot wins
    ref = synth.copy_tree(t)
    rng = np.random.default_rng(5)
    ids = np.concatenate([np.array([0, 1, 2, 3, 4, 5, 6, 7, 7, 1499, 1, 8, 9, 10], np.int32),
                          rng.integers(0, 1500, 1400).astype(np.int32)])
    ids[24], ids[25] = -1, 1500
    dt = api.DeviceTree(t)
    sel = dt.select(torch.from_numpy(ids).cuda(), c_puct=1.5, vl_value=3, apply_vl=False).cpu().numpy()
    want = np.full(len(ids), -1, np.int32)
    ok = (ids >= 0) & (ids < 1500)
    want[ok] = oracle.puct_select(ref, ids[ok], c_puct=1.5, vl_value=3, apply_vl=False)
    assert np.array_equal(sel, want)
    assert sel[0] == -1 and sel[1] == nc - 1
    # with virtual loss applied, whole tree
    sel2 = dt.select(c_puct=1.5, vl_value=3, apply_vl=True).cpu().numpy()
    sel2_ref = oracle.puct_select(ref, c_puct=1.5, vl_value=3, apply_vl=True)
    assert np.array_equal(sel2, sel2_ref) and np.array_equal(dt.host("VL"), ref["VL"])


def test_select_staged_path_with_node_ids(api, oracle):
    """Launches of >= 1024 entries on rows of <= 256 slots take the shared-memory staged
    kernel: node list with repeats and out-of-range ids, with and without virtual loss."""
    import torch
    t = synth.make_selection_tree(2048, 225, seed=23)
    t["legal_bits"][5] = 0
    t["W"][9, :225] = np.nan
    rng = np.random.default_rng(4)
    ids = rng.integers(0, 2048, 5000).astype(np.int32)
    ids[17], ids[18], ids[19], ids[20] = -1, 2048, 5, 9
    dt = api.DeviceTree(t)
    sel = dt.select(torch.from_numpy(ids).cuda(), c_puct=1.5, vl_value=3, apply_vl=False).cpu().numpy()
    want = np.full(len(ids), -1, np.int32)
    ok = (ids >= 0) & (ids < 2048)
    want[ok] = oracle.puct_select(synth.copy_tree(t), ids[ok], c_puct=1.5, vl_value=3, apply_vl=False)
    assert np.array_equal(sel, want)
    assert api.device_error_code() == 0
    # distinct nodes with virtual loss applied: state matches the oracle exactly
    ids = rng.permutation(2048)[:1500].astype(np.int32)
    ref = synth.copy_tree(t)
    sel = dt.select(torch.from_numpy(ids).cuda(), c_puct=1.5, vl_value=3, apply_vl=True).cpu().numpy()
    assert np.array_equal(sel, oracle.puct_select(ref, ids, c_puct=1.5, vl_value=3, apply_vl=True))
    assert np.array_equal(dt.host("VL"), ref["VL"])


def test_select_with_a_mask_array_that_is_only_4_byte_aligned(api, oracle):
    """The existence-mask array may be a slice of a larger buffer: 4-byte alignment is all the ABI
    asks of it.  A large launch then runs on the direct kernel (the staged one copies mask rows in
    16-byte units) and gives the same indices."""
    import ctypes as C
    import torch
    t = synth.make_selection_tree(2048, 225, seed=31)
    dt = api.DeviceTree(t)
    mw = t["legal_bits"].shape[1]
    holder = torch.zeros(2048 * mw + 8, dtype=torch.int32, device="cuda")
    shifted = holder[1:1 + 2048 * mw]                               # base + 4 bytes
    shifted.copy_(dt.t["legal_bits"].reshape(-1))
    assert shifted.data_ptr() % 16 == 4
    dt.view.legal_bits = shifted.data_ptr()
    sel = dt.select(c_puct=1.5, vl_value=3, apply_vl=False).cpu().numpy()
    assert np.array_equal(sel, oracle.puct_select(synth.copy_tree(t), c_puct=1.5, vl_value=3, apply_vl=False))
    # the statistics arrays do need 16 bytes: an argument check, nothing is launched
    dt.view.N = dt.t["N"].data_ptr() + 4
    with pytest.raises(api.Error) as e:
        dt.select(c_puct=1.5, vl_value=3, apply_vl=False)
    assert e.value.code == 1


def test_vl_revert_clamps_at_zero(api, oracle):
    import torch
    t = synth.make_selection_tree(128, 225, seed=22, vl_max=2)
    ref = synth.copy_tree(t)
    sel = torch.from_numpy(np.random.default_rng(0).integers(0, 225, 128).astype(np.int32)).cuda()
    dt = api.DeviceTree(t)
    dt.vl_revert(sel, 3)                                    # counters are 0..2: every one clamps to 0
    oracle.vl_revert(ref, sel.cpu().numpy(), 3)
    assert np.array_equal(dt.host("VL"), ref["VL"])
    dt.vl_apply(sel, 5); oracle.vl_apply(ref, sel.cpu().numpy(), 5)
    dt.vl_apply(sel, 0); dt.vl_apply(sel, -2)               # ignored, as the reference ignores amount <= 0
    assert np.array_equal(dt.host("VL"), ref["VL"])


def make_linked_tree(n_trees, depth_nodes, nc, seed):
    """A forest where each tree is a chain-with-branches: node ids allocated
    breadth-first, roughly half of the legal edges expanded."""
    rng = np.random.default_rng(seed)
    n_nodes = n_trees * depth_nodes
    t = synth.make_selection_tree(n_nodes, nc, seed=seed)
    child = np.full((n_nodes, t["N"].shape[1]), -1, np.int32)
    for tr in range(n_trees):
        base = tr * depth_nodes
        nxt = 1
        for local in range(depth_nodes):
            node = base + local
            legal = np.nonzero(np.unpackbits(t["legal_bits"][node].view(np.uint8), bitorder="little")[:nc])[0]
            for s in rng.permutation(legal)[: max(1, len(legal) // 2)]:
                if nxt >= depth_nodes:
                    break
                child[node, s] = base + nxt
                nxt += 1
    t["child_node"] = child
    roots = (np.arange(n_trees) * depth_nodes).astype(np.int32)
    return t, roots


def test_traverse_and_backup_bit_exact(api, oracle):
    import torch
    t, roots = make_linked_tree(16, 40, 225, seed=31)
    ref = synth.copy_tree(t)
    dt = api.DeviceTree(t)
    paths, plen = dt.traverse(torch.from_numpy(roots).cuda(), sims_per_tree=12, c_puct=1.5, vl_value=3, max_depth=16)
    rp, rl = oracle.traverse(ref, roots, 12, 1.5, 3, 16)
    assert np.array_equal(plen.cpu().numpy(), rl)
    assert np.array_equal(paths.cpu().numpy(), rp)
    assert np.array_equal(dt.host("VL"), ref["VL"])
    # backup with values that are exact in fp32 sums (multiples of 1/8) so that the order of
    # the atomic adds cannot change W
    vals = (np.random.default_rng(1).integers(-8, 9, len(rl)) / 8.0).astype(np.float32)
    dt.backup(paths, plen, torch.from_numpy(vals).cuda(), vl_value=3)
    oracle.backup(ref, rp, rl, vals, 3)
    assert np.array_equal(dt.host("N"), ref["N"]) and np.array_equal(dt.host("VL"), ref["VL"])
    assert np.array_equal(dt.host("node_visits"), ref["node_visits"])
    assert np.allclose(dt.host("W"), ref["W"], atol=1e-4)


def test_set_priors_bit_exact(api, oracle):
    import torch
    t = synth.make_selection_tree(64, 225, seed=41)
    ref = synth.copy_tree(t)
    rng = np.random.default_rng(2)
    ids = rng.permutation(64)[:20].astype(np.int32)
    pol = rng.uniform(-0.2, 1.2, (20, 225)).astype(np.float32)   # values outside [0,1] get clamped
    dt = api.DeviceTree(t)
    dt.set_priors(torch.from_numpy(ids).cuda(), torch.from_numpy(pol).cuda())
    oracle.set_priors(ref, ids, pol)
    assert np.array_equal(dt.host("P"), ref["P"])


def test_bad_arguments_are_reported(api):
    import ctypes as C
    t = synth.make_selection_tree(8, 225, seed=1)
    dt = api.DeviceTree(t)
    dt.view.pitch = 227                                       # not a multiple of 4
    with pytest.raises(api.Error) as e:
        dt.select()
    assert e.value.code == 1
    assert api.lib().ob200_launch_puct_select(None, None, 0, C.c_float(1.0), 0, 0, None, None) == 1
