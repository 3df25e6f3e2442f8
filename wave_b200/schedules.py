"""Names of the reference's manual MXFP4 schedules.

In the reference each function returns a schedule that software-pipelines the AMD kernel
(wave_lang/kernel/wave/schedules/gemm_mxfp4_double_buffer.py:42,284,519,726,1102,1471,1781):
global->LDS prefetch against LDS->register loads and MFMAs, with ping-pong and stagger variants.
The B200 kernels have their pipeline built in (TMA producer warp, tcgen05 issuer warp, epilogue
warps, 4 to 10 shared-memory stages, two accumulators in tensor memory), so these return a token
that `wave_compile` accepts and ignores.
"""

from dataclasses import dataclass, field


@dataclass(frozen=True)
class MXFP4Schedule:
    name: str
    args: tuple = field(default_factory=tuple)


def get_mxfp4_dbuf_schedule(use_stagger: bool = True, k_partitions: int = 2):
    return MXFP4Schedule("dbuf", (use_stagger, k_partitions))


def get_mxfp4_dbuf_pingpong_schedule(use_stagger: bool = True, *args, **kwargs):
    return MXFP4Schedule("dbuf_pingpong", (use_stagger,))


def get_mxfp4_dbuf_pingpong_schedule_Bshuffled(use_stagger: bool = True, *args, **kwargs):
    return MXFP4Schedule("dbuf_pingpong_Bshuffled", (use_stagger,))


def get_mxfp4_dbuf_pingpong_schedule_Bshuffled_lds(use_stagger: bool = True, *args, **kwargs):
    return MXFP4Schedule("dbuf_pingpong_Bshuffled_lds", (use_stagger,))


def get_mxfp4_dbuf_mixed_pingpong_schedule(use_stagger: bool = True):
    return MXFP4Schedule("dbuf_mixed_pingpong", (use_stagger,))


def get_mxfp4_dbuf_mixed_pingpong_shuffle_schedule(use_stagger: bool = True):
    return MXFP4Schedule("dbuf_mixed_pingpong_shuffle", (use_stagger,))


def get_mxfp4_asymmetric_schedule(*args, **kwargs):
    return MXFP4Schedule("asymmetric", tuple(args))
