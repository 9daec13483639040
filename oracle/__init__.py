"""CPU oracle for the block-quantized matmul path (test infrastructure only).

``oracle_c`` is the C restatement of the reference's CPU algorithm, ``oracle_np`` an
independent NumPy twin, ``build_oracle`` the build recipes.  The shipped library never
imports this package.
"""
