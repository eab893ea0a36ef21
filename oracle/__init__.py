"""CPU restatement of the reference algorithms on the generation-step hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the `evox_b200` package imports this; only `tests/`,
`__graft_entry__.smoke()` and the `cpu_baseline` / `--impl reference` legs of `bench.py` do,
as the checker and as the timed CPU baseline. Each function cites the reference source it
restates (EMI-Group/evox v1.3.0, paths relative to `src/evox/`). The restatements are written
with eager torch CPU ops because the reference itself is eager torch: the same ATen CPU kernels
give the same roundings. `tests/golden/` pins them against outputs of the reference itself.
"""
