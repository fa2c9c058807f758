"""helix_b200: the Helix dense-kernel generator / autotuner hot path, built for sm_100a.

``helix_b200.ops`` is the operator front-end over ``libhelix_b200.so``;
``helix_b200/scripts`` mirrors the reference's ``scripts/`` tree (same module,
function and CLI names).  Importing the package does not load CUDA; calling an
operator without the built library raises (there is no fallback path).
"""
__version__ = "1.0"
