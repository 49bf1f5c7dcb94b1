"""Weights from the reference project's checkpoints.

The reference saves its network with torch::serialize::OutputArchive
(ResNetModel::save, reference src/nn/resnet_model.cpp:813-828); such a file is a
TorchScript archive whose parameters and buffers carry the module's names
("input_conv.weight", "res_blocks.3.bn1.running_var", ...).  This module reads it
with the Python torch that is installed anyway, and writes the flat file that
B200Network::load (omoknuni_small_b200/adapter/b200_network.h) and capi.Net.load
take:  repeated { uint32 name_len, name, uint64 numel, float32 data[numel] }.

The reference's factory renames "model.pt" to e.g. "model_gomoku_15x15.pt" before
loading (src/nn/neural_network_factory.cpp:84-105); pass the file that exists.

    python -m omoknuni_small_b200.checkpoint model_gomoku_15x15.pt model_b200.bin
"""
import struct
import sys

import numpy as np


def load_reference_checkpoint(path):
    """name -> float32 numpy array (original shape) for every parameter and buffer."""
    import torch
    m = torch.jit.load(str(path), map_location="cpu")
    out = {}
    for name, t in list(m.named_parameters()) + list(m.named_buffers()):
        if name.endswith("num_batches_tracked"):
            continue
        out[name] = t.detach().to(torch.float32).contiguous().numpy()
    return out


def write_flat(path, tensors):
    with open(path, "wb") as f:
        for name, a in tensors.items():
            a = np.ascontiguousarray(a, np.float32).ravel()
            f.write(struct.pack("<I", len(name)) + name.encode() + struct.pack("<Q", a.size) + a.tobytes())


def read_flat(path):
    out = {}
    with open(path, "rb") as f:
        while True:
            head = f.read(4)
            if len(head) < 4:
                break
            (n,) = struct.unpack("<I", head)
            name = f.read(n).decode()
            (numel,) = struct.unpack("<Q", f.read(8))
            out[name] = np.frombuffer(f.read(4 * numel), np.float32).copy()
    return out


def infer_config(tensors):
    """Network shape from the tensor shapes: the arguments of ResNetModel's
    constructor (src/nn/resnet_model.cpp:51-53) plus the two head widths."""
    stem = np.asarray(tensors["input_conv.weight"])
    filters, cin = stem.shape[0], stem.shape[1] if stem.ndim == 4 else None
    if cin is None:
        raise ValueError("flat files lose shapes; infer the configuration from the checkpoint itself")
    blocks = 1 + max([int(k.split(".")[1]) for k in tensors if k.startswith("res_blocks.")] + [-1])
    pc = np.asarray(tensors["policy_conv.weight"]).shape[0]
    vc = np.asarray(tensors["value_conv.weight"]).shape[0]
    policy_size, k_p = np.asarray(tensors["policy_fc.weight"]).shape
    board = int(round((k_p // pc) ** 0.5))
    hidden = np.asarray(tensors["value_fc1.weight"]).shape[0]
    return dict(input_channels=int(cin), board_size=board, blocks=blocks, filters=int(filters),
                policy_size=int(policy_size), policy_head_ch=int(pc), value_head_ch=int(vc), value_hidden=int(hidden))


def main(argv):
    if len(argv) != 3:
        print(__doc__)
        return 2
    tensors = load_reference_checkpoint(argv[1])
    write_flat(argv[2], tensors)
    print(f"{len(tensors)} tensors, {sum(a.size for a in tensors.values())} values -> {argv[2]}")
    print(infer_config(tensors))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
