"""Measured throughput of every candidate configuration on a few shapes, next to the cost model's pick
(reference: scripts/Ampere_FP16/candidate_performance_curve.py:6-44).

The reference numbers candidates in dictionary order and spawns one executable per candidate; here the
candidates are the dictionary's kernel keys the model rates applicable to the shape (finite predicted
time), run in process.  Lines keep the reference's wording, with the candidate's own id.
"""
import os

import _bootstrap  # noqa: F401

root_path = os.getcwd()

# one shape of each kind the reference's script looks at (its literal list: candidate_performance_curve.py:42):
# ragged M on square weights, small with K not a multiple of 8, tall with ragged N, very wide with tiny K
DEFAULT_SHAPES = [(500, 1024, 1024), (128, 512, 1000), (5000, 712, 2048), (32, 50000, 104)]


def candidates(prof_dict, M, N, K):
    """[(id, key, predicted seconds)] in dictionary order, ids counted over kernel keys from 1."""
    from helix_b200 import harness
    out, idx = [], 0
    for k in prof_dict:
        if len(k) != 6:
            continue
        idx += 1
        if k[0] == 0 and min(M, N) > 8:
            continue
        t = harness.predicted_time(prof_dict, k, M, N, K)
        if t < float("inf"):
            out.append((idx, k, t))
    return out


def get_all_candidate_performance(prof_dict, M, N, K, out=print):
    from helix_b200 import harness
    cand = candidates(prof_dict, M, N, K)
    min_id, min_config, _ = min(cand, key=lambda c: c[2])
    out(f'Best candidate id: {min_id}, config = {min_config}')
    rows = []
    for idx, k, _ in cand:
        tflops = 2 * M * N * K / 1e12 / harness.time_key_f16(k, M, N, K)
        rows.append((idx, k, tflops))
        out(f'candidate id: {idx}, flops = {tflops} Tflops')
    return min_id, rows


if __name__ == "__main__":
    from helix_b200 import costmodel
    prof_dict = costmodel.load(f'{root_path}/build/prof_dict/Ampere_FP16_cost_model.dict')

    for M, N, K in DEFAULT_SHAPES:
        get_all_candidate_performance(prof_dict, M, N, K)
