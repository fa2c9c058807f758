"""Shape suites of the sweeps (role of the reference's scripts/utils/get_benchmark_shape_list.py:1-49).

Same four entry points, tuple conventions and contents as the reference -- GEMM units are (M, N, K);
convolution units are (batch, IC, H, W, OC, kH, kW, stride, pad).  What follows from an architecture's
dimensions (the transformer linear layers over the sequence-length sweep, the classifier layers over the
batch sweep) is generated; the reference's literal tables (DeepBench and GNN GEMMs, the convolution layer
lists, the AlexNet / ResNet / GoogLeNet op-sets) are data and live in shape_tables.json beside this file
(written by make_shape_tables.py).  HELIX_EXTRA_GEMM_SHAPES / HELIX_EXTRA_CONV_SHAPES may point at a JSON
file with further tuples to append to the op-level lists.  The benchmark's own model-level configuration
(BERT-base at batch 16, sequence 512 with its batched attention GEMMs, and the 53 ResNet-50 convolutions
at batch 32) lives in helix_b200/workloads.py.
"""
import json
import os

# token counts of the sequence-length sweep (60 values between 2 and 1949)
TOKEN_COUNTS = [2, 13, 31, 53, 73, 101, 127, 151, 179, 199, 233, 263, 283, 317, 353, 383, 419, 443, 467, 503, 547, 577,
                607, 641, 661, 701, 739, 769, 811, 839, 877, 911, 947, 983, 1019, 1049, 1087, 1109, 1153, 1193, 1229,
                1277, 1297, 1321, 1381, 1429, 1453, 1487, 1521, 1559, 1597, 1621, 1663, 1697, 1739, 1783, 1823, 1871,
                1902, 1949]
CNN_BATCHES = [1, 4, 8, 12, 16, 20, 24, 28, 32, 36, 40, 44, 48, 52, 56, 60, 64]


_TABLES = None


def _table(name):
    global _TABLES
    if _TABLES is None:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "shape_tables.json")) as f:
            _TABLES = json.load(f)
    return [tuple(row) for row in _TABLES[name]]


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
    return transformer + cnn + _table("gemm_deepbench") + _table("gemm_gnn") + _extra("HELIX_EXTRA_GEMM_SHAPES")


def get_llm_opset_MNKList():
    h, f = 768, 3072
    bert_nk = [(h, h)] * 49 + [(h, f)] * 12 + [(f, h)] * 12                    # 12 x (Q, K, V, O) + pooler, FFN
    llama2_nk = [(12288, 4096), (4096, 4096), (11008, 4096), (4096, 11008)]
    gpt2_nk = [(h, 3 * h)] * 24 + [(f, h)] * 48 + [(h, f)] * 24
    bert = [(m, n, k) for m in TOKEN_COUNTS for (n, k) in bert_nk]
    llama2 = [(m, n, k) for m in TOKEN_COUNTS for (n, k) in llama2_nk]
    gpt2 = [(m, n, k) for m in TOKEN_COUNTS for (n, k) in gpt2_nk]
    return bert, llama2, gpt2


def get_conv_op_shape_list():
    cnn = [(batch,) + shape for batch in CNN_BATCHES for shape in _table("conv_layers")]
    return cnn + _table("conv_deepbench") + _extra("HELIX_EXTRA_CONV_SHAPES")


def get_cnn_opset_shape_List():
    alexnet = [(batch,) + shape for batch in CNN_BATCHES for shape in _table("opset_alexnet")]
    resnet = [(batch,) + shape for batch in CNN_BATCHES for shape in _table("opset_resnet")]
    googlenet = [(batch,) + shape for batch in CNN_BATCHES for shape in _table("opset_googlenet")]
    return alexnet, resnet, googlenet
