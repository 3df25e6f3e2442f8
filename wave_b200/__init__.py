"""wave_b200: the MXFP4 scaled-GEMM path of Wave's kernel templates, on B200 (sm_100a).

    from wave_b200 import get_tagged_mxfp4_gemm, wave_compile, bf16
    kernel, options = get_tagged_mxfp4_gemm((M, N, K), output_dtype=bf16)
    gemm = wave_compile(options, kernel)
    gemm(a, a_scale, b, b_scale, c)      # torch CUDA tensors, c written in place

Computation happens in libwave_b200.so (hand-written tcgen05 / TMA kernels) behind the C ABI of
include/wave_b200.h; there is no CPU or PyTorch fallback.
"""

from .compile import (SchedulingType, ScaledGemmKernel, WaveCompileOptions, get_default_arch,  # noqa: F401
                      set_default_run_config, wave_compile)
from .constraints import ScaledMMAType  # noqa: F401
from .lang import (GLOBAL_ADDRESS_SPACE, SHARED_ADDRESS_SPACE, TORCH_DTYPE_TO_WAVE, bf16, f32, i8)  # noqa: F401
from .mxfp_utils import (SCALE_GROUP_SIZE, PackedScales, b_preshuffle, e8m0_shuffle,  # noqa: F401
                         generate_gemm_afp4wfp4_inputs, mxfp4_dequant, quantize_mxfp4)
from .schedules import (get_mxfp4_asymmetric_schedule, get_mxfp4_dbuf_mixed_pingpong_schedule,  # noqa: F401
                        get_mxfp4_dbuf_mixed_pingpong_shuffle_schedule, get_mxfp4_dbuf_pingpong_schedule,
                        get_mxfp4_dbuf_pingpong_schedule_Bshuffled, get_mxfp4_dbuf_pingpong_schedule_Bshuffled_lds,
                        get_mxfp4_dbuf_schedule)
from .templates import (get_broadcasted_scale_gemm_mxfp4, get_scaled_gemm_kernel, get_scaled_gemm_mxfp8_kernel, get_tagged_mxfp4_gemm, get_tagged_mxfp4_gemm_preshuffle_b,  # noqa: F401
                        get_tagged_mxfp4_gemm_preshuffle_b_wide_store, get_tagged_mxfp4_gemm_preshuffle_scales,
                        get_tagged_mxfp4_gemm_preshuffle_scales_and_B, get_tagged_splitk_mxfp4_gemm,
                        get_tagged_splitk_mxfp4_gemm_preshuffle_b, get_tagged_splitk_mxfp4_gemm_preshuffle_scales)

from .nn import MXFP4Linear  # noqa: F401,E402
from .moe import (MXFP4ExpertMLP, get_silu_and_mul_kernel, moe_align_block_size, silu_and_mul)  # noqa: F401,E402

__version__ = "0.1.0"
