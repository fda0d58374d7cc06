"""Generates tests/golden/small_cnn.npz from the reference's OWN C library: the outputs of the small CNN
of the first benchmark configuration (seed 0), computed node by node by oracle/graph.py on
oracle/_ref/tensor_ops_ref.so.  Run where the reference sources are available:

    python tests/golden/make_graph_golden.py

The graph is built by onnx_translator_b200.nn.small_cnn (constructing nodes needs no GPU); only the
two graph outputs are stored (prob [1,10] and the side branch [1,16,32,32], 64 KB)."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from oracle import graph as oracle_graph  # noqa: E402
from onnx_translator_b200 import nn  # noqa: E402


def main():
    graph, x = nn.small_cnn(seed=0)
    prob, side = oracle_graph.run(graph, oracle.HostOracle("ref"), x)
    np.savez_compressed(os.path.join(HERE, "small_cnn.npz"), prob=prob, side=side)
    print("prob", prob.shape, float(prob.sum()), "side", side.shape)


if __name__ == "__main__":
    main()
