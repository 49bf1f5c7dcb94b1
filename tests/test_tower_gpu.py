"""The tensor-core convolution layer and the whole network against fp32
references, through the C ABI.

Tolerances.  One layer: inputs and weights are bf16-exact, accumulation is
fp32, the output is rounded to bf16 once, so |err| <= 2^-8 * |y| + 1e-5.
Whole network: policy logits within 2e-2 and value within 1e-2 (max-abs) of the
fp32 forward for the reference module's own initialisation and for seeded
weights with random BatchNorm statistics in the default bf16 storage; for the
Kaiming-normal benchmark weights the bound holds with fp16 storage
(test_network_kaiming_normal_benchmark_weights_f16) and is missed by bf16 storage
(test_network_kaiming_normal_benchmark_weights_bf16_gap says by how much)."""
import numpy as np
import pytest

from omoknuni_small_b200 import synth
from test_oracle import load_net_golden_a, load_net_golden_b

pytestmark = pytest.mark.gpu

POLICY_TOL, VALUE_TOL = 2e-2, 1e-2


@pytest.fixture(scope="module")
def api(lib):
    from omoknuni_small_b200 import capi
    return capi


def bf16_round(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def f16_round(a):
    return np.ascontiguousarray(a, np.float32).astype(np.float16).astype(np.float32)


def conv_case(api, B, S, cin_real, cin, residual, relu, seed, cout=64, dtype=0, scale=1.0, wscale=0.1):
    import torch
    import torch.nn.functional as F
    rng = np.random.default_rng(seed)
    rnd = f16_round if dtype == 1 else bf16_round
    x = rnd(rng.normal(0, scale, (B, cin_real, S, S)).astype(np.float32))
    w = rnd(rng.normal(0, wscale, (cout, cin_real, 3, 3)).astype(np.float32))
    bias = rng.normal(0, 0.5, cout).astype(np.float32)
    res = rnd(rng.normal(0, 1, (B, cout, S, S)).astype(np.float32)) if residual else None
    y = F.conv2d(torch.from_numpy(x), torch.from_numpy(w), padding=1).numpy() + bias[None, :, None, None]
    if residual:
        y = y + res
    if relu:
        y = np.maximum(y, 0)
    xd = torch.from_numpy(api.planes_to_board_tensor_host(x, cin, dtype).view(np.int16)).cuda()
    rd = torch.from_numpy(api.planes_to_board_tensor_host(res, cout, dtype).view(np.int16)).cuda() if residual else None
    wd = torch.from_numpy(api.pack_conv3x3(w, None, cin, dtype).view(np.int16)).cuda()
    bd = torch.from_numpy(bias).cuda()
    # pre-fill the output with a pattern: the kernel must overwrite padding positions with zero
    out = torch.full((int(api.lib().ob200_board_tensor_bytes(S, B, cout)) // 2,), 0x3F80, dtype=torch.int16, device="cuda")
    PT = api.board_positions(S, B)
    o2 = out.view(PT, cout)
    o2[:api.GUARD] = 0
    o2[PT - api.GUARD:] = 0
    api.conv3x3(xd, wd, bd, rd, B, S, cin, cout, relu, out=out, dtype=dtype)
    torch.cuda.synchronize()
    assert api.device_error_code() == 0
    got, pad_zero = api.board_tensor_to_planes(out.cpu().numpy().view(np.uint16), S, B, cout, dtype)
    return got, y, pad_zero


@pytest.mark.parametrize("B,S,cin_real,cin,residual,relu", [
    (1, 15, 64, 64, False, False),
    (2, 15, 64, 64, True, True),
    (3, 15, 17, 64, False, True),      # the stem: 17 planes in a 64-channel tensor
    (37, 15, 64, 64, True, True),      # more tiles than fit one wave of 4 stages per CTA? (74 tiles)
    (700, 15, 64, 64, True, True),     # 1400 tiles: every CTA loops, stages and accumulators wrap
    (5, 9, 64, 64, True, True),        # 10x10 grid: tiles straddle boards
    (4, 19, 64, 64, False, True),      # 20x20 grid
    (9, 5, 64, 64, True, False),
])
def test_conv3x3_layer(api, B, S, cin_real, cin, residual, relu):
    got, want, pad_zero = conv_case(api, B, S, cin_real, cin, residual, relu, seed=B * 100 + S)
    err = np.abs(got - want)
    tol = np.abs(want) * 2.0 ** -8 + 1e-5
    bad = np.argwhere(err > tol)
    assert bad.size == 0, f"{len(bad)} of {err.size} elements off; first {bad[:5].tolist()}; max err {err.max():.4g}"
    assert pad_zero, "padding / guard positions of the output are not zero"


@pytest.mark.parametrize("B,S,cin_real,cin,cout,residual,relu", [
    (1, 15, 128, 128, 128, False, False),
    (2, 19, 128, 128, 128, True, True),      # Go tower layer
    (3, 19, 17, 64, 128, False, True),       # Go stem: 17 planes in a 64-channel tensor
    (40, 19, 128, 128, 128, True, True),     # 125 tiles: the last work unit holds a single tile
    (5, 8, 119, 128, 256, False, True),      # chess stem: 119 planes in a 128-channel tensor
    (6, 8, 256, 256, 256, True, True),       # chess tower layer: two 128-channel halves
    (700, 8, 256, 256, 256, True, True),     # 444 work units: every CTA loops, all rings wrap
    (300, 19, 128, 128, 128, True, True),    # 938 tiles
])
def test_conv3x3_layer_wide(api, B, S, cin_real, cin, cout, residual, relu):
    """Towers of 128 / 256 channels (streamed-weight kernel)."""
    got, want, pad_zero = conv_case(api, B, S, cin_real, cin, residual, relu, seed=B * 100 + S + cout, cout=cout)
    err = np.abs(got - want)
    tol = np.abs(want) * 2.0 ** -8 + 1e-4
    bad = np.argwhere(err > tol)
    assert bad.size == 0, f"{len(bad)} of {err.size} elements off; first {bad[:5].tolist()}; max err {err.max():.4g}"
    assert pad_zero, "padding / guard positions of the output are not zero"


@pytest.mark.parametrize("B,S,cin_real,cin,cout,residual,relu", [
    (2, 15, 64, 64, 64, True, True),
    (3, 15, 17, 64, 64, False, True),        # the stem
    (700, 15, 64, 64, 64, True, True),       # every CTA loops
    (5, 9, 64, 64, 64, True, False),
    (2, 19, 128, 128, 128, True, True),      # the streamed-weight kernel
    (6, 8, 256, 256, 256, True, True),
])
def test_conv3x3_layer_f16(api, B, S, cin_real, cin, cout, residual, relu):
    """The same layer with fp16 storage (OB200_DTYPE_F16): inputs and weights fp16-exact, fp32
    accumulation, one rounding to fp16 (11 significant bits)."""
    got, want, pad_zero = conv_case(api, B, S, cin_real, cin, residual, relu, seed=B * 100 + S + cout, cout=cout, dtype=1)
    err = np.abs(got - want)
    tol = np.abs(want) * 2.0 ** -11 + 1e-4
    bad = np.argwhere(err > tol)
    assert bad.size == 0, f"{len(bad)} of {err.size} elements off; first {bad[:5].tolist()}; max err {err.max():.4g}"
    assert pad_zero, "padding / guard positions of the output are not zero"


def test_conv3x3_f16_saturates_instead_of_overflowing(api):
    """fp16 storage ends at 65,504.  Inputs of magnitude ~1,000 times weights of magnitude ~2 over 576
    products push many sums beyond that: the stored outputs must be clamped to +-65,504 (+65,504 / 0 behind a ReLU), never
    inf or NaN, so that one outsized activation does not poison everything downstream."""
    for relu in (False, True):
        got, want, pad_zero = conv_case(api, 3, 15, 64, 64, False, relu, seed=99, dtype=1, scale=1000.0, wscale=2.0)
        assert np.isfinite(got).all()
        over = np.abs(want) > 65504.0
        assert over.mean() > 0.05, "the case must actually overflow"
        assert np.array_equal(got[over], np.sign(want[over]) * 65504.0)
        fine = np.abs(want) < 60000.0
        assert np.abs(got[fine] - want[fine]).max() <= 65504.0 * 2.0 ** -10
        assert pad_zero


def make_net(api, w, cfg, max_batch, dtype=0):
    return api.Net(cfg["cin"], cfg["S"], cfg["blocks"], cfg["F"], cfg["A"], cfg["pc"], cfg["vc"], 256, max_batch,
                   policy_kind=cfg.get("kind", 0), tower_dtype=dtype).load(w)


def mixed_planes(B, S, C, scalar_planes, seed):
    """Binary planes (p = 0.1) followed by `scalar_planes` planes uniform in [0, 1]."""
    rng = np.random.default_rng(seed)
    x = (rng.random((B, C, S, S)) < 0.1).astype(np.float32)
    if scalar_planes:
        x[:, C - scalar_planes:] = rng.random((B, scalar_planes, S, S)).astype(np.float32)
    return x


WIDE_NETS = [
    # Go 19x19 shape: 128 filters, policy 362, 2 / 1-channel heads
    ("go19_f128", dict(cin=17, S=19, blocks=4, F=128, A=362, pc=2, vc=1), 12, 0),
    # the reference's own head widths on a 128-filter tower
    ("go19_f128_heads32", dict(cin=17, S=19, blocks=2, F=128, A=362, pc=32, vc=32), 5, 0),
    # 15x15 with 256 filters and 19 planes
    ("gomoku15_f256", dict(cin=19, S=15, blocks=2, F=256, A=225, pc=2, vc=1), 9, 0),
    # chess shape: 119 planes (7 real-valued), 256 filters, 73 policy planes -> 4672 logits
    ("chess8_f256_planes", dict(cin=119, S=8, blocks=3, F=256, A=4672, pc=73, vc=1, kind=1), 37, 7),
    ("chess8_f128_planes", dict(cin=119, S=8, blocks=2, F=128, A=4672, pc=73, vc=1, kind=1), 6, 7),
]


@pytest.mark.parametrize("name,cfg,B,scalar", WIDE_NETS, ids=[n[0] for n in WIDE_NETS])
def test_network_wide_towers(api, name, cfg, B, scalar):
    """Towers of 128 / 256 filters (streamed-weight kernel), FC and convolution-plane policy
    heads, against the fp32 forward; libtorch-default initialisation with random BatchNorm."""
    from oracle import net_ref
    shapes = synth.net_tensor_shapes(cfg["S"], cfg["cin"], cfg["F"], cfg["blocks"], cfg["A"], cfg["pc"], cfg["vc"],
                                     policy_planes=cfg.get("kind", 0) == 1)
    w = synth.make_weights(shapes, seed=11, init="torch_default", bn="random")
    x = mixed_planes(B, cfg["S"], cfg["cin"], scalar, seed=2000 + B)
    ref_logits, ref_v = net_ref.forward(w, x)
    net = make_net(api, w, cfg, B + 3)
    logits, v = net.infer_planes(x, api.OUT_LOGITS)
    assert logits.shape == ref_logits.shape
    assert np.abs(logits - ref_logits).max() <= POLICY_TOL, np.abs(logits - ref_logits).max()
    assert np.abs(v - ref_v).max() <= VALUE_TOL
    probs, _ = net.infer_planes(x, api.OUT_PROBS)
    assert np.abs(probs - net_ref.softmax(ref_logits)).max() <= 1e-3 and np.allclose(probs.sum(1), 1, atol=1e-5)


def test_network_wide_tower_full_depth(api):
    """Go shape at the benchmark's depth (20 blocks x 128 filters, 41 tensor-core layers in a row)
    with the libtorch-default initialisation and random BatchNorm statistics, at the standard
    tolerances.  (Kaiming-normal weights with identity BatchNorm double the residual stream's
    variance per block: over 20 blocks the logits reach the hundreds and tanh saturates, which
    tests nothing.)"""
    from oracle import net_ref
    cfg = dict(cin=17, S=19, blocks=20, F=128, A=362, pc=2, vc=1)
    shapes = synth.net_tensor_shapes(19, 17, 128, 20, 362, 2, 1)
    w = synth.make_weights(shapes, seed=43, init="torch_default", bn="random")
    x = mixed_planes(6, 19, 17, 0, seed=77)
    ref_logits, ref_v = net_ref.forward(w, x)
    net = make_net(api, w, cfg, 8)
    logits, v = net.infer_planes(x, api.OUT_LOGITS)
    f_err, fv_err = np.abs(logits - ref_logits).max(), np.abs(v - ref_v).max()
    print(f"go 20x128: max|logit| {np.abs(ref_logits).max():.3f}, max|value| {np.abs(ref_v).max():.3f}; device vs fp32 {f_err:.5f} / {fv_err:.5f}")
    assert np.abs(ref_logits).max() > 0.05          # the comparison is not vacuous
    assert f_err <= POLICY_TOL and fv_err <= VALUE_TOL


def test_network_matches_reference_golden_default_init(api):
    """The reference module with its own libtorch initialisation (fixture (a))."""
    from oracle import net_ref
    cfg, w, x, logp, value = load_net_golden_a()
    net = make_net(api, w, cfg, 16)
    logits, v = net.infer_planes(x, api.OUT_LOGITS)
    assert np.abs(net_ref.log_softmax(logits) - logp).max() <= POLICY_TOL
    assert np.abs(v - value).max() <= VALUE_TOL
    probs, v2 = net.infer_planes(x, api.OUT_PROBS)
    assert np.abs(probs - np.exp(logp)).max() <= 1e-3 and np.allclose(probs.sum(1), 1, atol=1e-5)
    assert np.array_equal(v, v2)


def test_network_matches_reference_golden_15x15(api):
    """15x15, 10 blocks, reference 32/32 heads, seeded weights + random BatchNorm (fixture (b))."""
    from oracle import net_ref
    w, x, logp, value = load_net_golden_b()
    cfg = dict(cin=17, S=15, blocks=10, F=64, A=225, pc=32, vc=32)
    net = make_net(api, w, cfg, 8)
    logits, v = net.infer_planes(x, api.OUT_LOGITS)
    assert np.abs(net_ref.log_softmax(logits) - logp).max() <= POLICY_TOL
    assert np.abs(v - value).max() <= VALUE_TOL


@pytest.mark.parametrize("heads", [(2, 1), (32, 32)])
def test_network_torch_default_init_benchmark_shape(api, heads):
    """Benchmark network shape with the distribution the reference's C++ model is born with."""
    from oracle import net_ref
    shapes = synth.net_tensor_shapes(15, 17, 64, 10, 225, heads[0], heads[1])
    w = synth.make_weights(shapes, seed=3, init="torch_default", bn="identity")
    x = synth.make_stone_planes(64, 15, 17, seed=1001)
    ref_logits, ref_v = net_ref.forward(w, x)
    net = make_net(api, w, dict(cin=17, S=15, blocks=10, F=64, A=225, pc=heads[0], vc=heads[1]), 64)
    logits, v = net.infer_planes(x, api.OUT_LOGITS)
    assert np.abs(logits - ref_logits).max() <= POLICY_TOL
    assert np.abs(v - ref_v).max() <= VALUE_TOL


def kaiming_case():
    from oracle import net_ref
    shapes = synth.net_tensor_shapes(15, 17, 64, 10, 225, 2, 1)
    w = synth.make_weights(shapes, seed=42, init="kaiming_normal", bn="identity")
    x = synth.make_stone_planes(256, 15, 17, seed=1000)
    return w, x, net_ref.forward(w, x)


def test_network_kaiming_normal_benchmark_weights_f16(api):
    """The benchmark's weights (Kaiming-normal convolutions with ReLU gain, identity BatchNorm,
    2/1-channel heads) at the stated tolerance: logits within 2e-2, value within 1e-2 of the fp32
    forward.  With identity BatchNorm the residual stream doubles in variance per block and 21 layers of
    8-bit significands drift several 1e-2 from fp32 (next test); fp16 storage (11 bits, activations
    peak near 32, far inside its range) holds the bound, and is what the benchmark runs."""
    from oracle import net_ref
    w, x, (ref_logits, ref_v) = kaiming_case()
    net = make_net(api, w, dict(cin=17, S=15, blocks=10, F=64, A=225, pc=2, vc=1), 256, dtype=api.DTYPE_F16)
    logits, v = net.infer_planes(x, api.OUT_LOGITS)
    assert net.tower_path() == 2
    emu_logits, emu_v = net_ref.forward_f16(w, x)
    f_err, fv_err = np.abs(logits - ref_logits).max(), np.abs(v - ref_v).max()
    print(f"kaiming-normal, fp16 storage: max|logit| {np.abs(ref_logits).max():.2f}; device vs fp32 {f_err:.4f} / {fv_err:.4f}; "
          f"fp16 emulation vs fp32 {np.abs(emu_logits - ref_logits).max():.4f} / {np.abs(emu_v - ref_v).max():.4f}")
    assert f_err <= POLICY_TOL and fv_err <= VALUE_TOL
    assert (logits.argmax(1) == ref_logits.argmax(1)).mean() >= 0.98
    probs, _ = net.infer_planes(x, api.OUT_PROBS)
    assert np.abs(probs - net_ref.softmax(ref_logits)).max() <= 1e-3


def test_network_kaiming_normal_benchmark_weights_bf16_gap(api):
    """The same weights in the default bf16 storage MISS the 2e-2 / 1e-2 bound: the fp32-arithmetic
    emulation of bf16 storage (oracle/net_ref.forward_bf16) is itself about 0.09 (logits) / 0.02 (value)
    from fp32, and so is the device.  This test documents that gap and holds the kernels to the
    emulation (the device's gap to fp32 must not exceed the emulation's by more than half, and the
    preferred move must agree wherever fp32's margin is clear); networks with such weights belong on
    OB200_DTYPE_F16."""
    from oracle import net_ref
    w, x, (ref_logits, ref_v) = kaiming_case()
    emu_logits, emu_v = net_ref.forward_bf16(w, x)
    net = make_net(api, w, dict(cin=17, S=15, blocks=10, F=64, A=225, pc=2, vc=1), 256)
    logits, v = net.infer_planes(x, api.OUT_LOGITS)
    k_err, kv_err = np.abs(logits - emu_logits).max(), np.abs(v - emu_v).max()
    f_err, fv_err = np.abs(logits - ref_logits).max(), np.abs(v - ref_v).max()
    e_err = np.abs(emu_logits - ref_logits).max()
    print(f"kaiming-normal, bf16 storage: max|logit| {np.abs(ref_logits).max():.2f}; device vs bf16 emulation {k_err:.4f} / {kv_err:.4f}; "
          f"device vs fp32 {f_err:.4f} / {fv_err:.4f}; bf16 emulation vs fp32 {e_err:.4f}")
    ev_err = np.abs(emu_v - ref_v).max()
    assert f_err <= 1.5 * e_err + POLICY_TOL and fv_err <= 1.5 * ev_err + VALUE_TOL
    assert k_err <= 2 * e_err and kv_err <= 2 * ev_err + VALUE_TOL
    # the preferred move agrees wherever the fp32 margin exceeds twice the gap
    order = np.argsort(ref_logits, 1)
    rows = np.arange(len(order))
    margin = ref_logits[rows, order[:, -1]] - ref_logits[rows, order[:, -2]]
    assert (logits.argmax(1) == order[:, -1])[margin > 2 * f_err].all()


@pytest.mark.parametrize("name,cfg,B", [
    ("gomoku15_f64_heads32", dict(cin=19, S=15, blocks=3, F=64, A=225, pc=32, vc=32), 20),
    ("go19_f64", dict(cin=17, S=19, blocks=2, F=64, A=362, pc=2, vc=1), 9),         # too large to stay resident
    ("go19_f128", dict(cin=17, S=19, blocks=2, F=128, A=362, pc=2, vc=1), 7),
    ("chess8_f256_planes", dict(cin=119, S=8, blocks=2, F=256, A=4672, pc=73, vc=1, kind=1), 11),
])
def test_network_f16_storage_other_shapes(api, name, cfg, B):
    """fp16 storage on the other tower paths: head kernel instead of the riding-along heads, the
    per-layer / cooperative 64-filter kernels (19x19), the streamed-weight kernel and the
    convolution-plane policy head."""
    from oracle import net_ref
    shapes = synth.net_tensor_shapes(cfg["S"], cfg["cin"], cfg["F"], cfg["blocks"], cfg["A"], cfg["pc"], cfg["vc"],
                                     policy_planes=cfg.get("kind", 0) == 1)
    w = synth.make_weights(shapes, seed=12, init="torch_default", bn="random")
    x = mixed_planes(B, cfg["S"], cfg["cin"], 7 if cfg["cin"] == 119 else 0, seed=2100 + B)
    ref_logits, ref_v = net_ref.forward(w, x)
    net = make_net(api, w, cfg, B + 3, dtype=api.DTYPE_F16)
    logits, v = net.infer_planes(x, api.OUT_LOGITS)
    assert np.abs(logits - ref_logits).max() <= POLICY_TOL / 4, np.abs(logits - ref_logits).max()
    assert np.abs(v - ref_v).max() <= VALUE_TOL / 4


def pick_tower(monkeypatch, which):
    """Pins the tower path a network handle created afterwards will use: "layers" (a launch per
    layer), "fused" (one cooperative launch, tiles handed over through flags) or "resident" (one
    launch, boards kept in shared memory)."""
    if which == "resident":
        monkeypatch.delenv("OB200_TOWER_FUSED", raising=False)
        monkeypatch.setenv("OB200_TOWER_RESIDENT", "1")
    else:
        monkeypatch.setenv("OB200_TOWER_RESIDENT", "0")
        monkeypatch.setenv("OB200_TOWER_FUSED", "2" if which == "fused" else "0")


@pytest.mark.parametrize("S,blocks,B", [(15, 1, 1), (15, 1, 2), (15, 2, 3), (9, 2, 5), (10, 1, 40), (11, 1, 40), (13, 4, 700),
                                        (15, 3, 150), (15, 10, 300), (15, 10, 1024), (15, 13, 10)])
def test_resident_tower_equals_layer_by_layer(api, monkeypatch, S, blocks, B):
    """The board-resident tower (activations never leave shared memory) runs the same arithmetic in
    the same order as the launch-per-layer path: outputs must be bit-identical.  One and two
    boards per CTA, an odd number of boards per CTA, boards of one tile (up to 10x10) and of two."""
    shapes = synth.net_tensor_shapes(S, 17, 64, blocks, S * S, 2, 1)
    w = synth.make_weights(shapes, seed=5, init="torch_default", bn="random")
    x = synth.make_stone_planes(B, S, 17, seed=4000 + B)
    outs = []
    for which in ("resident", "layers"):
        pick_tower(monkeypatch, which)
        net = make_net(api, w, dict(cin=17, S=S, blocks=blocks, F=64, A=S * S, pc=2, vc=1), B)
        before = api.counters()["kernel_launches"]
        logits, v = net.infer_planes(x, api.OUT_LOGITS)
        launches = api.counters()["kernel_launches"] - before
        logits2, v2 = net.infer_planes(x, api.OUT_LOGITS)
        assert np.array_equal(logits, logits2) and np.array_equal(v, v2)
        assert net.tower_path() == (2 if which == "resident" else 0)
        outs.append((logits, v, launches))
        net.close()
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    # 1 tower launch instead of 1 + 2 * blocks, and the heads' 1x1 convolutions ride along in it
    assert outs[0][2] == outs[1][2] - 2 * blocks - 1
    assert api.device_error_code() == 0


@pytest.mark.parametrize("S,blocks,B", [(15, 10, 300), (9, 2, 5), (15, 3, 149)])
def test_f16_tower_paths_bit_identical(api, monkeypatch, S, blocks, B):
    """fp16 storage: the board-resident tower, the cooperative single-launch tower and the
    launch-per-layer path are the same arithmetic in the same order, bit for bit."""
    shapes = synth.net_tensor_shapes(S, 17, 64, blocks, S * S, 2, 1)
    w = synth.make_weights(shapes, seed=6, init="torch_default", bn="random")
    x = synth.make_stone_planes(B, S, 17, seed=4100 + B)
    outs = []
    for which, path in (("resident", 2), ("fused", 1), ("layers", 0)):
        pick_tower(monkeypatch, which)
        net = make_net(api, w, dict(cin=17, S=S, blocks=blocks, F=64, A=S * S, pc=2, vc=1), B, dtype=api.DTYPE_F16)
        outs.append(net.infer_planes(x, api.OUT_LOGITS))
        assert net.tower_path() == path
        net.close()
    for o in outs[1:]:
        assert np.array_equal(outs[0][0], o[0]) and np.array_equal(outs[0][1], o[1])
    assert api.device_error_code() == 0


@pytest.mark.parametrize("B", [3, 300, 1100])
def test_fused_tower_equals_layer_by_layer(api, monkeypatch, B):
    """The single-launch tower (CTAs walk the layers, tiles hand over through flags) and the
    launch-per-layer path run the same arithmetic: outputs must be bit-identical.  Batches with
    fewer tiles than CTAs, a few tiles per CTA, and 15 tiles per CTA."""
    shapes = synth.net_tensor_shapes(15, 17, 64, 10, 225, 2, 1)
    w = synth.make_weights(shapes, seed=5, init="torch_default", bn="random")
    x = synth.make_stone_planes(B, 15, 17, seed=4000 + B)
    outs = []
    for which in ("fused", "layers"):
        pick_tower(monkeypatch, which)
        net = make_net(api, w, dict(cin=17, S=15, blocks=10, F=64, A=225, pc=2, vc=1), B)
        before = api.counters()["kernel_launches"]
        logits, v = net.infer_planes(x, api.OUT_LOGITS)
        launches = api.counters()["kernel_launches"] - before
        logits2, v2 = net.infer_planes(x, api.OUT_LOGITS)          # flags of the first call must not leak into the second
        assert np.array_equal(logits, logits2) and np.array_equal(v, v2)
        outs.append((logits, v, launches))
        net.close()
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    assert outs[0][2] == outs[1][2] - 20                           # 1 tower launch instead of 21
    assert api.device_error_code() == 0


@pytest.mark.parametrize("which,B,iters", [("fused", 1024, 400), ("fused", 700, 200), ("resident", 1024, 400),
                                           ("resident", 301, 200), ("resident", 100, 300)])
def test_single_launch_tower_repeats_bit_identically(api, monkeypatch, which, B, iters):
    """Hundreds of back-to-back single-launch towers on one input: every result equals the first
    (a tile read before its producer wrote it, or a flag left over from an earlier launch, would
    show up as a different output sooner or later)."""
    import torch
    pick_tower(monkeypatch, which)
    shapes = synth.net_tensor_shapes(15, 17, 64, 10, 225, 2, 1)
    w = synth.make_weights(shapes, seed=42, init="kaiming_normal")
    net = api.Net(17, 15, 10, 64, 225, 2, 1, 256, B).load(w)
    _, hist, nh, tm = synth.make_gomoku_games(B, 15, seed=B)
    dh, dn, dt = (torch.from_numpy(a).cuda() for a in (hist, nh, tm))
    bt = api.encode_gomoku(dh, dn, dt, 15, 17, 64)
    pol = torch.empty((B, 225), device="cuda")
    val = torch.empty(B, device="cuda")
    net.forward_device(bt, B, pol, val, api.OUT_LOGITS)
    torch.cuda.synchronize()
    p0, v0 = pol.clone(), val.clone()
    different = torch.zeros((), dtype=torch.int64, device="cuda")
    for _ in range(iters):
        net.forward_device(bt, B, pol, val, api.OUT_LOGITS)
        different += (pol != p0).any() | (val != v0).any()
    torch.cuda.synchronize()
    net.close()
    assert int(different) == 0
    assert api.device_error_code() == 0


def test_resident_tower_hands_over_when_the_shape_does_not_fit(api, monkeypatch):
    """14 blocks = 29 layers of biases do not fit beside the boards in shared memory, a 19x19 board does
    not fit at all, 128 filters are another kernel: the handle then takes one of the other paths."""
    pick_tower(monkeypatch, "resident")
    for S, blocks, F in ((15, 14, 64), (19, 1, 64), (15, 1, 128)):
        shapes = synth.net_tensor_shapes(S, 17, F, blocks, S * S, 2, 1)
        w = synth.make_weights(shapes, seed=3, init="torch_default", bn="random")
        net = make_net(api, w, dict(cin=17, S=S, blocks=blocks, F=F, A=S * S, pc=2, vc=1), 4)
        net.infer_planes(synth.make_stone_planes(3, S, 17, seed=1), api.OUT_LOGITS)
        assert net.tower_path() in (0, 1)
        net.close()
    shapes = synth.net_tensor_shapes(15, 17, 64, 13, 225, 2, 1)
    net = make_net(api, synth.make_weights(shapes, seed=3, init="torch_default", bn="random"),
                   dict(cin=17, S=15, blocks=13, F=64, A=225, pc=2, vc=1), 4)
    net.infer_planes(synth.make_stone_planes(3, 15, 17, seed=1), api.OUT_LOGITS)
    assert net.tower_path() == 2
    net.close()
    assert api.device_error_code() == 0


@pytest.mark.parametrize("S,blocks,B,cin,which", [(9, 0, 5, 3, "fused"), (5, 1, 17, 17, "fused"), (30, 1, 3, 19, "fused"),
                                                    (19, 2, 70, 17, "fused"), (19, 2, 70, 17, "layers"), (7, 3, 1, 64, "fused"),
                                                    (9, 0, 5, 3, "resident"), (5, 1, 17, 17, "resident"), (7, 3, 1, 64, "resident"),
                                                    (15, 2, 149, 19, "resident"), (19, 1, 9, 17, "resident")])
def test_network_odd_shapes(api, monkeypatch, S, blocks, B, cin, which):
    """Board sizes from 5 to 30, a tower without blocks, 3 / 64 input planes, single boards; on each of
    the three tower paths (a 19x19 board does not fit the board-resident one, which then hands over to
    the others)."""
    from oracle import net_ref
    pick_tower(monkeypatch, which)
    A = S * S
    shapes = synth.net_tensor_shapes(S, cin, 64, blocks, A, 2, 1)
    w = synth.make_weights(shapes, seed=S + blocks, init="torch_default", bn="random")
    x = mixed_planes(B, S, cin, 0, seed=50 + S)
    ref_logits, ref_v = net_ref.forward(w, x, blocks=blocks)
    net = make_net(api, w, dict(cin=cin, S=S, blocks=blocks, F=64, A=A, pc=2, vc=1), B)
    logits, v = net.infer_planes(x, api.OUT_LOGITS)
    assert np.abs(logits - ref_logits).max() <= POLICY_TOL and np.abs(v - ref_v).max() <= VALUE_TOL
    assert api.device_error_code() == 0


def test_forward_device_in_a_captured_graph(api):
    """ob200_net_forward_device captured into a CUDA graph and replayed on new inputs gives what
    direct calls give (the single-launch tower keeps a per-launch epoch on the host, so a capturing
    stream must get the per-layer kernels)."""
    import torch
    B = 700                                            # a batch at which direct calls use the single launch
    shapes = synth.net_tensor_shapes(15, 17, 64, 4, 225, 2, 1)
    w = synth.make_weights(shapes, seed=9, init="torch_default", bn="random")
    net = make_net(api, w, dict(cin=17, S=15, blocks=4, F=64, A=225, pc=2, vc=1), B)
    xs = [synth.make_stone_planes(B, 15, 17, seed=7000 + i) for i in range(3)]
    bts = [api.planes_to_board_tensor(torch.from_numpy(x).cuda(), net.input_tensor_channels()) for x in xs]
    pol = torch.empty((B, 225), dtype=torch.float32, device="cuda")
    val = torch.empty(B, dtype=torch.float32, device="cuda")
    direct = []
    for bt in bts:
        net.forward_device(bt, B, pol, val, api.OUT_LOGITS)
        torch.cuda.synchronize()
        direct.append((pol.cpu().numpy().copy(), val.cpu().numpy().copy()))
    static_in = bts[0].clone()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        net.forward_device(static_in, B, pol, val, api.OUT_LOGITS)      # warm-up outside capture
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(g):
        net.forward_device(static_in, B, pol, val, api.OUT_LOGITS)
    for bt, (p_ref, v_ref) in zip(bts, direct):
        static_in.copy_(bt)
        g.replay()
        g.replay()                                     # a second replay must not see the first one's state
        torch.cuda.synchronize()
        assert np.array_equal(pol.cpu().numpy(), p_ref) and np.array_equal(val.cpu().numpy(), v_ref)
    assert api.device_error_code() == 0


def test_gomoku_inference_end_to_end(api, oracle):
    """Host move histories -> encoder -> tower -> heads, against oracle encoder + fp32 forward,
    including a batch smaller than max_batch after a larger one (buffer reuse)."""
    from oracle import net_ref
    shapes = synth.net_tensor_shapes(15, 19, 64, 10, 225, 32, 32)
    w = synth.make_weights(shapes, seed=8, init="torch_default", bn="random")
    net = api.Net(19, 15, 10, 64, 225, 32, 32, 256, 300).load(w)
    for B, seed in ((300, 1), (5, 2), (129, 3)):
        games, hist, nh, tm = synth.make_gomoku_games(B, 15, seed=seed)
        planes = oracle.gomoku_encode(hist, nh, tm, 15, 19)
        ref_logits, ref_v = net_ref.forward(w, planes)
        probs, v = net.infer_gomoku(hist, nh, tm, api.OUT_PROBS)
        assert np.abs(probs - net_ref.softmax(ref_logits)).max() <= 1e-3
        assert np.abs(v - ref_v).max() <= VALUE_TOL
        assert np.allclose(probs.sum(1), 1, atol=1e-5) and (probs >= 0).all()


def test_bounded_wait_reports_and_context_survives(api):
    """A device-side wait that runs out raises the error word (no trap, no hang); the host reads
    and clears it, the host-buffer inference call turns it into OB200_ERR_TIMEOUT, and the
    context keeps working."""
    import torch
    from oracle import net_ref
    shapes = synth.net_tensor_shapes(15, 17, 64, 2, 225, 2, 1)
    w = synth.make_weights(shapes, seed=2, init="torch_default")
    net = api.Net(17, 15, 2, 64, 225, 2, 1, 256, 8).load(w)
    x = synth.make_stone_planes(8, 15, 17, seed=5)
    good, _ = net.infer_planes(x, api.OUT_LOGITS)
    assert api.device_error_code() == 0
    api.check(api.lib().ob200_debug_bounded_wait(2000, None))
    assert api.device_error_code() == 9          # reported ...
    assert api.device_error_code() == 0          # ... and cleared by the read
    api.check(api.lib().ob200_debug_bounded_wait(2000, None))
    torch.cuda.synchronize()                     # the handle's own stream does not wait for the default stream
    with pytest.raises(api.Error) as e:          # the inference call notices it on its own
        net.infer_planes(x, api.OUT_LOGITS)
    assert e.value.code == 6
    again, _ = net.infer_planes(x, api.OUT_LOGITS)
    assert np.array_equal(good, again) and api.device_error_code() == 0
    ref_logits, _ = net_ref.forward(w, x)
    assert np.abs(again - ref_logits).max() <= POLICY_TOL


@pytest.mark.parametrize("F,blocks,B", [(64, 10, 1024), (128, 3, 600)])
def test_network_batch_invariance(api, F, blocks, B):
    """Size-independent property at the benchmark's batch: a position's outputs do not depend on
    what else is in the batch, nor on where its tiles fall (whole batch vs uneven chunks, bit for bit)."""
    shapes = synth.net_tensor_shapes(15, 17, F, blocks, 225, 2, 1)
    w = synth.make_weights(shapes, seed=6, init="torch_default", bn="random")
    x = synth.make_stone_planes(B, 15, 17, seed=6000)
    net = make_net(api, w, dict(cin=17, S=15, blocks=blocks, F=F, A=225, pc=2, vc=1), B)
    logits, v = net.infer_planes(x, api.OUT_LOGITS)
    cuts = [0, 1, 130, 131 + B // 3, B]
    parts = [net.infer_planes(x[a:b], api.OUT_LOGITS) for a, b in zip(cuts[:-1], cuts[1:])]
    assert np.array_equal(logits, np.concatenate([p[0] for p in parts]))
    assert np.array_equal(v, np.concatenate([p[1] for p in parts]))


def test_inference_argument_errors(api):
    shapes = synth.net_tensor_shapes(15, 17, 64, 1, 225, 2, 1)
    w = synth.make_weights(shapes, seed=1, init="torch_default")
    net = api.Net(17, 15, 1, 64, 225, 2, 1, 256, 4)
    with pytest.raises(api.Error) as e:
        net.infer_planes(np.zeros((1, 17, 15, 15), np.float32))
    assert e.value.code == 4                                   # weights not finalised
    missing = dict(w)
    del missing["policy_fc.bias"]
    with pytest.raises(api.Error) as e:
        api.Net(17, 15, 1, 64, 225, 2, 1, 256, 4).load(missing)
    assert e.value.code == 4 and "policy_fc.bias" in str(e.value)
    net.load(w)
    with pytest.raises(api.Error) as e:
        net.infer_planes(np.zeros((5, 17, 15, 15), np.float32))
    assert e.value.code == 7                                   # beyond max_batch
    with pytest.raises(api.Error):
        api.Net(17, 15, 1, 96, 225)                            # tower width outside this build


def test_two_batches_in_flight_give_the_same_results(api):
    """submit / wait with two calls pending (the results of one batch travel back while the next one computes)
    and the one-call form from four threads at once: every batch gets exactly the outputs of a plain
    synchronous call; a third submit without a wait is refused with a status."""
    import threading
    import torch
    shapes = synth.net_tensor_shapes(15, 17, 64, 3, 225, 2, 1)
    w = synth.make_weights(shapes, seed=8, init="torch_default", bn="random")
    B, n_batches = 200, 7
    net = make_net(api, w, dict(cin=17, S=15, blocks=3, F=64, A=225, pc=2, vc=1), 256)
    batches = [synth.make_gomoku_games(B, 15, seed=600 + i)[1:] for i in range(n_batches)]
    want = [net.infer_gomoku(h, nh, tm) for h, nh, tm in batches]
    # pinned and pageable output buffers alike
    for pinned in (True, False):
        outs = []
        for _ in range(n_batches):
            if pinned:
                p, v = torch.empty((B, 225), dtype=torch.float32).pin_memory(), torch.empty(B, dtype=torch.float32).pin_memory()
                outs.append((p.numpy(), v.numpy(), p, v))
            else:
                outs.append((np.empty((B, 225), np.float32), np.empty(B, np.float32)))
        tickets = []
        for i, (h, nh, tm) in enumerate(batches):
            if len(tickets) == 2:
                net.wait(tickets.pop(0))
            tickets.append(net.submit_gomoku(h, nh, tm, outs[i][:2]))
        with pytest.raises(api.Error) as e:                                  # both slots are pending here
            net.submit_gomoku(*batches[0], outs[0][:2])
        assert e.value.code == 4
        for t in tickets:
            net.wait(t)
        with pytest.raises(api.Error):
            net.wait(0)                                                      # nothing pending any more
        for i in range(n_batches):
            assert np.array_equal(outs[i][0], want[i][0]) and np.array_equal(outs[i][1], want[i][1]), i
    got = [None] * n_batches

    def worker(k):
        for i in range(k, n_batches, 4):
            got[i] = net.infer_gomoku(*batches[i])
    threads = [threading.Thread(target=worker, args=(k,)) for k in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for i in range(n_batches):
        assert np.array_equal(got[i][0], want[i][0]) and np.array_equal(got[i][1], want[i][1]), i
    assert api.device_error_code() == 0


@pytest.mark.parametrize("S,blocks,B,dtype,which", [(15, 2, 1, 0, "resident"), (15, 3, 300, 0, "resident"), (15, 10, 1024, 1, "resident"),
                                                    (15, 2, 149, 1, "resident"), (9, 2, 37, 0, "resident"), (13, 2, 450, 1, "resident"),
                                                    (15, 2, 300, 0, "layers"), (19, 1, 5, 1, "layers")])
def test_forward_from_move_histories_equals_encode_then_forward(api, monkeypatch, S, blocks, B, dtype, which):
    """ob200_net_forward_gomoku_device (the board-resident tower writes its own input planes from the move
    histories) against ob200_launch_encode_gomoku followed by ob200_net_forward_device: the same planes, so the
    same bits out - boards of one and two tiles, one to seven boards per CTA, both storage types, and the tower
    paths that run the encoder kernel themselves."""
    import torch
    pick_tower(monkeypatch, which)
    shapes = synth.net_tensor_shapes(S, 19, 64, blocks, S * S, 2, 1)
    w = synth.make_weights(shapes, seed=13, init="torch_default", bn="random")
    net = make_net(api, w, dict(cin=19, S=S, blocks=blocks, F=64, A=S * S, pc=2, vc=1), B, dtype=dtype)
    games, hist, nh, tm = synth.make_gomoku_games(B, S, seed=900 + B)
    dh, dn, dt = (torch.from_numpy(a).cuda() for a in (hist, nh, tm))
    outs = []
    for fused in (True, False):
        pol = torch.zeros((B, S * S), dtype=torch.float32, device="cuda")
        val = torch.zeros(B, dtype=torch.float32, device="cuda")
        if fused:
            net.forward_gomoku_device(dh, dn, dt, pol, val, api.OUT_LOGITS)
        else:
            bt = api.encode_gomoku(dh, dn, dt, S, 19, net.input_tensor_channels(), dtype)
            net.forward_device(bt, B, pol, val, api.OUT_LOGITS)
        torch.cuda.synchronize()
        outs.append((pol.cpu().numpy(), val.cpu().numpy()))
    assert net.tower_path() == (2 if which == "resident" else 0)
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    assert np.abs(outs[0][0]).max() > 0 and api.device_error_code() == 0
    # and through the host-buffer call
    pol_h, val_h = net.infer_gomoku(hist, nh, tm, api.OUT_LOGITS)
    assert np.array_equal(pol_h, outs[0][0]) and np.array_equal(val_h, outs[0][1])
