"""Shape suites of the benchmark configurations (pure Python, no device).

Mirrors the role of scripts/utils/get_benchmark_shape_list.py in the reference:
GEMM units are (M, N, K) tuples (batched ones (M, N, K, batch)); convolution
units use the reference's tuple order (batch, IC, H, W, OC, kH, kW, stride, pad)
(scripts/Ampere_FP16/benchmark_Ampere_FP16_conv.py:15).
"""


def bert_base_gemms(batch=16, seq=512, hidden=768, heads=12, ffn=3072, layers=12):
    """Every GEMM of a BERT-base encoder: per layer QKV, QK^T, PV, out-projection, FFN up/down."""
    tokens = batch * seq
    head_dim = hidden // heads
    per_layer = [
        ("qkv", (tokens, 3 * hidden, hidden)),
        ("qk", (seq, seq, head_dim, batch * heads)),
        ("pv", (seq, head_dim, seq, batch * heads)),
        ("out_proj", (tokens, hidden, hidden)),
        ("ffn_up", (tokens, ffn, hidden)),
        ("ffn_down", (tokens, hidden, ffn)),
    ]
    units = []
    for layer in range(layers):
        for name, shape in per_layer:
            units.append({"kind": "gemm", "name": f"bert.l{layer}.{name}", "shape": shape})
    return units


def resnet50_convs(batch=32, image=224):
    """The 53 convolutions of ResNet-50 v1.5 (stride on the 3x3) at `batch` x image x image."""
    units = []

    def add(name, ic, h, oc, k, stride, pad):
        units.append({"kind": "conv", "name": f"resnet50.{name}", "shape": (batch, ic, h, h, oc, k, k, stride, pad)})
        return (h + 2 * pad - k) // stride + 1

    h = add("stem", 3, image, 64, 7, 2, 3)          # 224 -> 112
    h = (h + 2 * 1 - 3) // 2 + 1                   # 3x3/2 max-pool, pad 1: 112 -> 56
    in_ch = 64
    for stage, (width, blocks) in enumerate([(64, 3), (128, 4), (256, 6), (512, 3)]):
        out_ch = width * 4
        for blk in range(blocks):
            stride = 2 if (blk == 0 and stage > 0) else 1
            tag = f"s{stage + 1}b{blk}"
            add(f"{tag}.conv1", in_ch, h, width, 1, 1, 0)
            h_out = add(f"{tag}.conv2", width, h, width, 3, stride, 1)
            add(f"{tag}.conv3", width, h_out, out_ch, 1, 1, 0)
            if blk == 0:
                add(f"{tag}.proj", in_ch, h, out_ch, 1, stride, 0)
            h = h_out
            in_ch = out_ch
    return units


def model_level_sweep(bert_batch=16, seq=512, resnet_batch=32):
    """Model-level sweep: BERT-base GEMMs followed by the ResNet-50 convolutions."""
    return bert_base_gemms(bert_batch, seq) + resnet50_convs(resnet_batch)


def unit_flops(unit):
    s = unit["shape"]
    if unit["kind"] == "gemm":
        M, N, K = s[:3]
        b = s[3] if len(s) > 3 else 1
        return 2.0 * M * N * K * b
    B, IC, H, W, OC, kh, kw, stride, pad = s
    Ho, Wo = (H + 2 * pad - kh) // stride + 1, (W + 2 * pad - kw) // stride + 1
    return 2.0 * B * Ho * Wo * OC * IC * kh * kw


def unit_bytes(unit):
    """Algorithmic bytes: every operand read once, the output written once (fp16)."""
    s = unit["shape"]
    if unit["kind"] == "gemm":
        M, N, K = s[:3]
        b = s[3] if len(s) > 3 else 1
        return 2.0 * b * (M * K + N * K + M * N)
    B, IC, H, W, OC, kh, kw, stride, pad = s
    Ho, Wo = (H + 2 * pad - kh) // stride + 1, (W + 2 * pad - kw) // stride + 1
    return 2.0 * (B * H * W * IC + OC * kh * kw * IC + B * Ho * Wo * OC)


def lpt_partition(costs, parts):
    """Longest-processing-time-first assignment of independent units to `parts` workers.

    Returns a list of index lists; deterministic (ties broken by index).
    """
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    loads = [0.0] * parts
    out = [[] for _ in range(parts)]
    for i in order:
        p = min(range(parts), key=lambda q: (loads[q], q))
        out[p].append(i)
        loads[p] += costs[i]
    for lst in out:
        lst.sort()
    return out
