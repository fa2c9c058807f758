"""Shape suites of the sweeps (role of the reference's scripts/utils/get_benchmark_shape_list.py:1-49).

Same four entry points and tuple conventions as the reference -- GEMM units are (M, N, K); convolution
units are (batch, IC, H, W, OC, kH, kW, stride, pad) -- but the lists are generated here from the
architectures' published layer dimensions instead of being stored as literals.  The reference
additionally appends DeepBench- and GNN-derived GEMM/conv literals to the op-level lists; those are not
reproduced: point HELIX_EXTRA_GEMM_SHAPES / HELIX_EXTRA_CONV_SHAPES at a JSON file with a list of tuples
to sweep any further shapes.  The benchmark's own model-level configuration (BERT-base at batch 16,
sequence 512 with its batched attention GEMMs, and the 53 ResNet-50 convolutions at batch 32) lives in
helix_b200/workloads.py.
"""
import json
import os

# token counts of the sequence-length sweep (60 values between 2 and 1949)
TOKEN_COUNTS = [2, 13, 31, 53, 73, 101, 127, 151, 179, 199, 233, 263, 283, 317, 353, 383, 419, 443, 467, 503, 547, 577,
                607, 641, 661, 701, 739, 769, 811, 839, 877, 911, 947, 983, 1019, 1049, 1087, 1109, 1153, 1193, 1229,
                1277, 1297, 1321, 1381, 1429, 1453, 1487, 1521, 1559, 1597, 1621, 1663, 1697, 1739, 1783, 1823, 1871,
                1902, 1949]
CNN_BATCHES = [1, 4, 8, 12, 16, 20, 24, 28, 32, 36, 40, 44, 48, 52, 56, 60, 64]


def _extra(env):
    path = os.environ.get(env)
    if not path:
        return []
    with open(path) as f:
        return [tuple(int(v) for v in row) for row in json.load(f)]


def _transformer_nk():
    """(N, K) of the linear layers of BERT-large, BERT-base / GPT-2, LLaMA-2 13B and 7B."""
    pairs = []
    h, f = 1024, 4096                       # BERT-large
    pairs += [(h, h), (f, h), (h, f)]
    h, f = 768, 3072                        # BERT-base / GPT-2 small
    pairs += [(h, 3 * h), (f, h), (h, f), (h, h)]
    pairs += [(4096, 4096)]
    h, f = 5120, 13824                      # LLaMA-2 13B: fused QKV, out-proj, FFN up / down
    pairs += [(3 * h, h), (h, h), (f, h), (h, f)]
    h, f = 4096, 11008                      # LLaMA-2 7B
    pairs += [(3 * h, h), (h, h), (f, h), (h, f)]
    return pairs


def get_gemm_op_MNKList():
    transformer = [(m, n, k) for m in TOKEN_COUNTS for (n, k) in _transformer_nk()]
    # fully connected layers of the CNN classifiers at batch 1..128
    fc_nk = [(12544, 120), (120, 80), (80, 10), (9216, 4096), (4096, 4096), (4096, 1000), (25088, 4096), (512, 1000),
             (1024, 1000), (25088, 1000)]
    cnn = [(m, n, k) for m in [1, 2, 4, 8, 16, 32, 64, 128] for (n, k) in fc_nk]
    return transformer + cnn + _extra("HELIX_EXTRA_GEMM_SHAPES")


def get_llm_opset_MNKList():
    h, f = 768, 3072
    bert_nk = [(h, h)] * 49 + [(h, f)] * 12 + [(f, h)] * 12                    # 12 x (Q, K, V, O) + pooler, FFN
    llama2_nk = [(12288, 4096), (4096, 4096), (11008, 4096), (4096, 11008)]
    gpt2_nk = [(h, 3 * h)] * 24 + [(f, h)] * 48 + [(h, f)] * 24
    bert = [(m, n, k) for m in TOKEN_COUNTS for (n, k) in bert_nk]
    llama2 = [(m, n, k) for m in TOKEN_COUNTS for (n, k) in llama2_nk]
    gpt2 = [(m, n, k) for m in TOKEN_COUNTS for (n, k) in gpt2_nk]
    return bert, llama2, gpt2


def _alexnet():
    return [(3, 224, 224, 96, 11, 11, 4, 0), (96, 26, 26, 256, 5, 5, 1, 2), (256, 12, 12, 384, 3, 3, 1, 1),
            (384, 12, 12, 384, 3, 3, 1, 1), (384, 12, 12, 256, 3, 3, 1, 1)]


def _resnet18_style():
    """3x3 stem at full resolution, then four stages of two basic blocks; stage changes by a strided 3x3 and a
    1x1 projection."""
    layers = [(3, 224, 224, 64, 3, 3, 1, 1)]
    ch, res = 64, 112
    layers += [(ch, res, res, ch, 3, 3, 1, 1)] * 4
    for _ in range(3):
        out, nres = ch * 2, res // 2
        layers += [(ch, res, res, out, 3, 3, 2, 1), (out, nres, nres, out, 3, 3, 1, 1), (ch, res, res, out, 1, 1, 2, 0),
                   (out, nres, nres, out, 3, 3, 1, 1), (out, nres, nres, out, 3, 3, 1, 1)]
        ch, res = out, nres
    return layers


def _googlenet():
    """Stem plus the nine inception modules (1x1, 3x3-reduce, 3x3, 5x5-reduce, 5x5, pool-projection)."""
    layers = [(3, 224, 224, 64, 7, 7, 2, 3), (64, 56, 56, 192, 3, 3, 1, 1)]
    modules = [  # (resolution, in, n1x1, n3x3r, n3x3, n5x5r, n5x5, pool)
        (28, 192, 64, 96, 128, 16, 32, 32), (28, 256, 128, 128, 192, 32, 96, 64),
        (14, 480, 192, 96, 208, 16, 48, 64), (14, 512, 160, 112, 224, 24, 64, 64), (14, 512, 128, 128, 256, 24, 64, 64),
        (14, 512, 112, 144, 288, 32, 64, 64), (14, 528, 256, 160, 320, 32, 128, 128),
        (7, 832, 256, 160, 320, 32, 128, 128), (7, 832, 384, 192, 384, 48, 128, 128)]
    for r, cin, n1, n3r, n3, n5r, n5, pp in modules:
        layers += [(cin, r, r, n1, 1, 1, 1, 0), (cin, r, r, n3r, 1, 1, 1, 0), (n3r, r, r, n3, 3, 3, 1, 1),
                   (cin, r, r, n5r, 1, 1, 1, 0), (n5r, r, r, n5, 5, 5, 1, 2), (cin, r, r, pp, 1, 1, 1, 0)]
    return layers


def get_conv_op_shape_list():
    without_batch = _alexnet() + _googlenet() + _resnet18_style()
    cnn = [(batch,) + shape for batch in CNN_BATCHES for shape in without_batch]
    return cnn + _extra("HELIX_EXTRA_CONV_SHAPES")


def get_cnn_opset_shape_List():
    alexnet = [(batch,) + shape for batch in CNN_BATCHES for shape in _alexnet()]
    resnet = [(batch,) + shape for batch in CNN_BATCHES for shape in _resnet18_style()]
    googlenet = [(batch,) + shape for batch in CNN_BATCHES for shape in _googlenet()]
    return alexnet, resnet, googlenet
