"""CPU oracle for the PrivateUse1 operator path -- TEST INFRASTRUCTURE ONLY.

Nothing in the product (the kernel library, the host extension, the Python
package) imports this package. It is used by tests/, by the smoke check and by
the benchmark's CPU-baseline leg as the checker and the timed CPU reference.

What the oracle is
------------------
The reference backend defines correctness of every operator as "equal to the
CPU kernel of the same ATen operator within a dtype tolerance": its run-time
op-check re-dispatches each op to DispatchKey::CPU and compares
(torch_gcu/csrc/aten/aot_ops/gcu_op_check.cpp:73-130,202-230; tolerances
torch_gcu/csrc/aten/op_debug_config.h:144-149), and its unit tests compare
against the CPU result of the same `torch.ops.aten.*` call
(test/op_test/gcu_op_test.py:49-135). The arithmetic itself lives in the closed
vendor library TopsAten (TopsRider v3.7.1, README.md:453-455), which is not in
the reference tree, so the oracle is PyTorch's CPU ATen, called directly
(`aten_cpu.py`), plus an independent plain-C restatement of the order-sensitive
integer/index algorithms (`seq_ref.c`) that pins ATen's accumulation order.

Pinning
-------
`tests/golden/` holds vectors produced in the build container by
`tests/golden/make_golden.py` from CPU ATen on the reference's own test cases
(shapes, seeds and tolerances read from test/op_test/test_binary_ops.py and
test/op_test/test_linear.py) and on small cases of every other operator. The
reference ships no golden files and pins no other operator of this path; for
those operators parity is pinned by ATen-vs-C-restatement agreement and the
committed vectors only.
"""
