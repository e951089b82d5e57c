"""Example programs against the AttentionEngine / LinearAttentionEngine API: the workloads the benchmark,
the smoke run and the parity tests use (softmax, sigmoid, relu, retention, MLA, decode patterns).  They are
written the way the reference's examples/*.py are; the package is named examples_b200 so that it does not
shadow the reference's own top-level ``examples`` package when both are importable."""
