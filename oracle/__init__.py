"""CPU oracle for the packed ternary linear path.  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the bench's CPU-baseline legs import this
package; the shipped package never does.  See ``bt_oracle.c`` for the parity
status of each function (integer path: parity unpinned by the reference's tests).
"""

from .oracle import (  # noqa: F401
    DT_F32,
    DT_F16,
    DT_BF16,
    build,
    ternarize,
    pack,
    pack_transposed,
    unpack,
    unpack_transposed,
    act_quant,
    gemm_i32,
    epilogue,
    linear_float,
    packed_forward_i8,
    packed_forward_i8_threaded,
    ref_python_forward,
    silu_mul_quant,
    add_rmsnorm_quant,
    exp_plain,
)
