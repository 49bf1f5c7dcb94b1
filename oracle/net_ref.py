"""TEST INFRASTRUCTURE: fp32 restatement of the reference network forward.

Follows alphazero::nn::ResNetModel::forward (reference
src/nn/resnet_model.cpp:104-237) and ResNetResidualBlock::forward (:43-49) with
torch CPU fp32 ops, taking weights under the reference's parameter names.  The
two head widths the reference hard-codes as 32 (:81-96) are read from the
weight shapes, so the same code covers the 2-channel / 1-channel heads of the
benchmark configuration.  Pinned against the reference's own class through
oracle/_ref/libref_net.so (tests/test_oracle.py) and the golden fixtures in
tests/golden/.
"""
import numpy as np
import torch
import torch.nn.functional as F

BN_EPS = 1e-5  # torch::nn::BatchNorm2dOptions default, used by the reference as is


def _bn(x, w, prefix):
    return F.batch_norm(x, w[prefix + ".running_mean"], w[prefix + ".running_var"], w[prefix + ".weight"],
                        w[prefix + ".bias"], training=False, eps=BN_EPS)


def forward(weights, planes, blocks=None, threads=0, return_tower=False):
    """weights: dict name -> numpy fp32 (reference names); planes [B,C,S,S] fp32.
    Returns (logits [B,A] before log-softmax, value [B] after tanh) as numpy."""
    if threads:
        torch.set_num_threads(threads)
    w = {k: torch.from_numpy(np.ascontiguousarray(v, np.float32)) for k, v in weights.items()}
    if blocks is None:
        blocks = 1 + max(int(k.split(".")[1]) for k in w if k.startswith("res_blocks."))
    with torch.no_grad():
        x = torch.from_numpy(np.ascontiguousarray(planes, np.float32))
        cin = w["input_conv.weight"].shape[1]
        if x.shape[1] != cin:  # :117-147 channel adaptation: copy min(C) channels into zeros
            y = torch.zeros(x.shape[0], cin, x.shape[2], x.shape[3])
            c = min(cin, x.shape[1])
            y[:, :c] = x[:, :c]
            x = y
        x = F.relu(_bn(F.conv2d(x, w["input_conv.weight"], padding=1), w, "input_bn"))       # :150
        for i in range(blocks):                                                                 # :43-49
            p = f"res_blocks.{i}."
            y = F.relu(_bn(F.conv2d(x, w[p + "conv1.weight"], padding=1), w, p + "bn1"))
            y = _bn(F.conv2d(y, w[p + "conv2.weight"], padding=1), w, p + "bn2")
            x = F.relu(y + x)
        tower = x
        if "policy_fc.weight" in w:
            pol = F.relu(_bn(F.conv2d(x, w["policy_conv.weight"]), w, "policy_bn"))               # :178
            logits = F.linear(pol.reshape(pol.shape[0], -1), w["policy_fc.weight"], w["policy_fc.bias"])  # :183-188
        else:   # convolutional policy head (not in the reference): planes flattened in NCHW order
            logits = F.conv2d(x, w["policy_conv.weight"], w["policy_conv.bias"]).reshape(x.shape[0], -1)
        val = F.relu(_bn(F.conv2d(x, w["value_conv.weight"]), w, "value_bn"))                 # :204
        val = F.relu(F.linear(val.reshape(val.shape[0], -1), w["value_fc1.weight"], w["value_fc1.bias"]))  # :214
        val = torch.tanh(F.linear(val, w["value_fc2.weight"], w["value_fc2.bias"]))          # :219
    out = (logits.numpy(), val.reshape(-1).numpy())
    return out + (tower.numpy(),) if return_tower else out


def log_softmax(logits):
    m = logits.max(1, keepdims=True)
    return logits - m - np.log(np.exp(logits - m).sum(1, keepdims=True))


def softmax(logits):
    return np.exp(log_softmax(logits))


def _bf16(t):
    return t.to(torch.bfloat16).to(torch.float32)


def _f16(t):
    # the device stores fp16 activations saturated at the largest finite value
    return t.clamp(-65504.0, 65504.0).to(torch.float16).to(torch.float32)


def forward_bf16(weights, planes, blocks=None):
    """forward_stored with bfloat16 storage (the device path's default)."""
    return forward_stored(weights, planes, blocks, _bf16)


def forward_f16(weights, planes, blocks=None):
    """forward_stored with float16 storage (the device path's OB200_DTYPE_F16)."""
    return forward_stored(weights, planes, blocks, _f16)


def forward_stored(weights, planes, blocks=None, _bf16=_bf16):
    """The same network with the storage precision of the device path, still in
    fp32 arithmetic on the CPU: BatchNorm folded into the convolution
    (w * gamma / sqrt(var + eps), shift as fp32 bias), folded tower weights and
    every stored activation rounded to the 16-bit storage type (`_bf16`: the
    rounding function), heads in fp32 on the tower output.  It says what the
    16-bit design computes; the gap between this and forward() is the price of
    the storage type, the gap between this and the device is kernel error."""
    w = {k: torch.from_numpy(np.ascontiguousarray(v, np.float32)) for k, v in weights.items()}
    if blocks is None:
        blocks = 1 + max([int(k.split(".")[1]) for k in w if k.startswith("res_blocks.")] + [-1])

    def fold(conv, bn):
        s = w[bn + ".weight"] / torch.sqrt(w[bn + ".running_var"] + BN_EPS)
        return w[conv + ".weight"] * s[:, None, None, None], w[bn + ".bias"] - w[bn + ".running_mean"] * s

    with torch.no_grad():
        x = torch.from_numpy(np.ascontiguousarray(planes, np.float32))
        cin = w["input_conv.weight"].shape[1]
        if x.shape[1] != cin:
            y = torch.zeros(x.shape[0], cin, x.shape[2], x.shape[3])
            c = min(cin, x.shape[1])
            y[:, :c] = x[:, :c]
            x = y
        x = _bf16(x)
        wf, b = fold("input_conv", "input_bn")
        x = _bf16(F.relu(F.conv2d(x, _bf16(wf), padding=1) + b[None, :, None, None]))
        for i in range(blocks):
            p = f"res_blocks.{i}."
            wf, b = fold(p + "conv1", p + "bn1")
            y = _bf16(F.relu(F.conv2d(x, _bf16(wf), padding=1) + b[None, :, None, None]))
            wf, b = fold(p + "conv2", p + "bn2")
            x = _bf16(F.relu(F.conv2d(y, _bf16(wf), padding=1) + b[None, :, None, None] + x))
        if "policy_fc.weight" in w:
            wf, b = fold("policy_conv", "policy_bn")
            pol = F.relu(F.conv2d(x, wf) + b[None, :, None, None])
            logits = F.linear(pol.reshape(pol.shape[0], -1), w["policy_fc.weight"], w["policy_fc.bias"])
        else:   # convolutional policy head: 16-bit weights on the tensor cores, fp32 accumulate and output
            logits = F.conv2d(x, _bf16(w["policy_conv.weight"]), w["policy_conv.bias"]).reshape(x.shape[0], -1)
        wf, b = fold("value_conv", "value_bn")
        val = F.relu(F.conv2d(x, wf) + b[None, :, None, None])
        val = F.relu(F.linear(val.reshape(val.shape[0], -1), w["value_fc1.weight"], w["value_fc1.bias"]))
        val = torch.tanh(F.linear(val, w["value_fc2.weight"], w["value_fc2.bias"]))
    return logits.numpy(), val.reshape(-1).numpy()
