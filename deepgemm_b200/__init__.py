"""deepgemm_b200: block-scaled FP8 / FP8xFP4 GEMMs for NVIDIA B200, behind the `deep_gemm` names.

`import deepgemm_b200 as deep_gemm` gives the operator surface of the reference's
deep_gemm/__init__.py:18-104 for the block-scaled GEMM family; every operator runs an
ahead-of-time built sm_100a kernel from libdeepgemm_b200.so through a C ABI.  There is no
CPU path: calling an operator without the library or a CUDA device raises RuntimeError.
"""
from . import utils, testing  # noqa: F401
from . import ops as _ops
from . import _lib
from .layout import (  # noqa: F401
    transform_sf_into_required_layout,
    get_tma_aligned_size,
    get_mn_major_tma_aligned_tensor,
    get_mn_major_tma_aligned_packed_ue8m0_tensor,
    get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor,
    set_mk_alignment_for_contiguous_layout,
    get_mk_alignment_for_contiguous_layout,
    get_theoretical_mk_alignment_for_contiguous_layout,
)
from .ops import (  # noqa: F401
    fp8_fp4_gemm_nt, fp8_fp4_gemm_nn, fp8_fp4_gemm_tn, fp8_fp4_gemm_tt,
    m_grouped_fp8_fp4_gemm_nt_contiguous, m_grouped_fp8_fp4_gemm_nn_contiguous,
    m_grouped_fp8_fp4_gemm_nt_masked, k_grouped_fp8_gemm_tn_contiguous, k_grouped_fp4_gemm_nt_contiguous,
)
from .einsum import fp8_einsum  # noqa: F401
from .bf16 import (  # noqa: F401
    bf16_gemm_nt, bf16_gemm_nn, bf16_gemm_tn, bf16_gemm_tt, m_grouped_bf16_gemm_nt_contiguous,
    m_grouped_bf16_gemm_nn_contiguous, m_grouped_bf16_gemm_nt_masked, k_grouped_bf16_gemm_tn_contiguous,
)

from . import mega  # noqa: F401,E402
from . import cast  # noqa: F401,E402
from .cast import per_token_cast_to_fp8_fused  # noqa: F401,E402
from .mega import (  # noqa: F401,E402
    SymmBuffer, get_symm_buffer_for_mega_moe, transform_weights_for_mega_moe, fp8_fp4_mega_moe,
    get_token_alignment_for_mega_moe, get_block_m_for_mega_moe, RouteWeightMode,
)

__version__ = "0.1.0"

# Aliases (csrc/apis/gemm.hpp:927-936 of the reference)
fp8_gemm_nt, fp8_gemm_nn, fp8_gemm_tn, fp8_gemm_tt = fp8_fp4_gemm_nt, fp8_fp4_gemm_nn, fp8_fp4_gemm_tn, fp8_fp4_gemm_tt
m_grouped_fp8_gemm_nt_contiguous = m_grouped_fp8_fp4_gemm_nt_contiguous
m_grouped_fp8_gemm_nn_contiguous = m_grouped_fp8_fp4_gemm_nn_contiguous
m_grouped_fp8_gemm_nt_masked = m_grouped_fp8_fp4_gemm_nt_masked
fp8_m_grouped_gemm_nt_masked = m_grouped_fp8_fp4_gemm_nt_masked
fp4_gemm_nt = fp8_fp4_gemm_nt
m_grouped_fp4_gemm_nt_contiguous = m_grouped_fp8_fp4_gemm_nt_contiguous
m_grouped_fp4_gemm_nt_masked = m_grouped_fp8_fp4_gemm_nt_masked


def k_grouped_fp8_gemm_nt_contiguous(*args, **kwargs):
    """The K-major (NT) form of the K-grouped FP8 GEMM exists for sm_90 only; on sm_100 the reference's dispatch
    ends in `Unsupported architecture` (csrc/apis/gemm.hpp:377-431).  Use k_grouped_fp8_gemm_tn_contiguous."""
    raise RuntimeError("Unsupported architecture: k_grouped_fp8_gemm_nt_contiguous is an sm_90 entry point; "
                       "sm_100 takes k_grouped_fp8_gemm_tn_contiguous")


class epilogue:  # namespace, as deep_gemm.epilogue (csrc/apis/epilogue_class.hpp:13-31 of the reference)
    Identity = _ops.Identity
    Alpha = _ops.Alpha
    FP8CastWithClamp = _ops.FP8CastWithClamp
    BF16StochasticRounding = _ops.BF16StochasticRounding


# Process-wide knobs (csrc/apis/config.hpp:8-48 of the reference)
def set_num_sms(num_sms: int) -> None:
    _lib.check(_lib.lib().dg_set_num_sms(int(num_sms)))


def get_num_sms() -> int:
    return int(_lib.lib().dg_get_num_sms())


def set_tc_util(tc_util: int) -> None:
    _lib.check(_lib.lib().dg_set_tc_util(int(tc_util)))


def get_tc_util() -> int:
    return int(_lib.lib().dg_get_tc_util())


_deterministic = False


def set_pdl(enable: bool) -> None:
    """Launch the GEMM, scale-packing and cast kernels with programmatic dependent launch: a kernel's set-up (barriers,
    tensor-memory allocation, descriptor prefetch) overlaps the tail of the kernel before it in the stream, and it
    waits in-kernel before reading anything that kernel wrote (csrc/apis/config.hpp:27-32 of the reference)."""
    _lib.check(_lib.lib().dg_set_pdl(int(bool(enable))))


def get_pdl() -> bool:
    return bool(_lib.lib().dg_get_pdl())


def use_deterministic_algorithms(enable: bool) -> None:
    """All kernels here are run-to-run deterministic; the flag is recorded only."""
    global _deterministic
    _deterministic = bool(enable)


def set_ignore_compile_dims(flag: bool) -> None:
    """Shapes are run-time arguments of ahead-of-time built kernels; nothing to ignore."""


def set_block_size_multiple_of(*_args, **_kwargs) -> None:
    """Accepted for compatibility."""


def init(*_args, **_kwargs) -> None:
    """The reference initialises its JIT here; this build has none."""


def shutdown() -> None:
    pass


check_status = _lib.check_status
