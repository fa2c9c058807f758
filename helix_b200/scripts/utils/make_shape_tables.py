"""Writes shape_tables.json (next to this file): the literal shape tables of the reference's
scripts/utils/get_benchmark_shape_list.py that cannot be derived from an architecture's dimensions -- the
DeepBench and GNN GEMM lists (:11, :13), the op-level convolution layer list and the DeepBench convolutions
(:32, :34), and the AlexNet / ResNet / GoogLeNet op-sets (:41-43).  The tables are data, not code: the
reference's functions are run with a tracer that records those local lists as they are built.

  HELIX_REFERENCE_TREE=<path to the reference checkout> python make_shape_tables.py
"""
import hashlib
import importlib.util
import json
import os
import sys

WANTED = {
    "get_gemm_op_MNKList": ["DeepBench_MNKList", "GNN_MNKList"],
    "get_conv_op_shape_list": ["CNN_shape_list_without_batch", "DeepBench_shape_list"],
    "get_cnn_opset_shape_List": ["AlexNet_MNKList_without_batch", "ResNet_MNKList_without_batch",
                                 "GoogleNet_MNKList_without_batch"],
}


def capture(module):
    got = {}

    def tracer(frame, event, arg):
        name = frame.f_code.co_name
        if name not in WANTED:
            return None

        def local(frame, event, arg):
            if event == "return":
                for var in WANTED[name]:
                    got[var] = [list(t) for t in frame.f_locals[var]]
            return local
        return local
    sys.settrace(tracer)
    try:
        out = {fn: getattr(module, fn)() for fn in list(WANTED) + ["get_llm_opset_MNKList"]}
    finally:
        sys.settrace(None)
    return got, out


def digest(lists):
    return hashlib.sha256(repr([[tuple(t) for t in lst] for lst in lists]).encode()).hexdigest()


def main():
    tree = os.environ.get("HELIX_REFERENCE_TREE")
    if not tree:
        raise SystemExit("set HELIX_REFERENCE_TREE to the reference checkout")
    spec = importlib.util.spec_from_file_location("ref_shape_list", os.path.join(tree, "scripts", "utils", "get_benchmark_shape_list.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    got, out = capture(mod)
    tables = {
        "gemm_deepbench": got["DeepBench_MNKList"], "gemm_gnn": got["GNN_MNKList"],
        "conv_layers": got["CNN_shape_list_without_batch"], "conv_deepbench": got["DeepBench_shape_list"],
        "opset_alexnet": got["AlexNet_MNKList_without_batch"], "opset_resnet": got["ResNet_MNKList_without_batch"],
        "opset_googlenet": got["GoogleNet_MNKList_without_batch"],
    }
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "shape_tables.json"), "w") as f:
        json.dump(tables, f, separators=(",", ":"))
        f.write("\n")
    print("sha256 of the four functions' outputs (pin these in the tests):")
    print("  gemm_op ", len(out["get_gemm_op_MNKList"]), digest([out["get_gemm_op_MNKList"]]))
    print("  llm     ", [len(x) for x in out["get_llm_opset_MNKList"]], digest(out["get_llm_opset_MNKList"]))
    print("  conv_op ", len(out["get_conv_op_shape_list"]), digest([out["get_conv_op_shape_list"]]))
    print("  cnn     ", [len(x) for x in out["get_cnn_opset_shape_List"]], digest(out["get_cnn_opset_shape_List"]))


if __name__ == "__main__":
    main()
