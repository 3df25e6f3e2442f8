"""Element-type and address-space tokens of the kernel templates.

Stand-ins for the reference's `tkl.f32` / `tkl.bf16` / `tkl.i8` data types
(wave_lang/kernel/lang/wave_types.py) and `SHARED_ADDRESS_SPACE` / `GLOBAL_ADDRESS_SPACE`
(wave_lang/kernel/lang/global_symbols.py), which the MXFP4 templates take as arguments. On B200
the address-space choice has no effect (operands always go through TMA into shared memory); the
tokens are accepted so that calls written against the reference keep working.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class DataType:
    name: str
    torch_dtype: torch.dtype

    def __repr__(self) -> str:
        return self.name


f32 = DataType("f32", torch.float32)
bf16 = DataType("bf16", torch.bfloat16)
i8 = DataType("i8", torch.int8)

# Same table as wave_lang/kernel/wave/utils/torch_utils.py TORCH_DTYPE_TO_WAVE, for the two output types.
TORCH_DTYPE_TO_WAVE = {torch.float32: f32, torch.bfloat16: bf16}


@dataclass(frozen=True)
class AddressSpace:
    name: str

    def __repr__(self) -> str:
        return self.name


GLOBAL_ADDRESS_SPACE = AddressSpace("GLOBAL_ADDRESS_SPACE")
SHARED_ADDRESS_SPACE = AddressSpace("SHARED_ADDRESS_SPACE")


def as_output_dtype(t) -> DataType:
    """Accept a DataType token or a torch dtype; only f32 and bf16 outputs exist
    (wave_lang/kernel/wave/templates/tagged_mxfp4_gemm.py:62-65)."""
    if isinstance(t, DataType):
        dt = t
    elif isinstance(t, torch.dtype) and t in TORCH_DTYPE_TO_WAVE:
        dt = TORCH_DTYPE_TO_WAVE[t]
    else:
        raise AssertionError(f"Unsupported output dtype: {t}")
    assert dt in (f32, bf16), f"Unsupported output dtype: {t}"
    return dt
