"""Per-kernel precision policy (Source/Public/Oa/Ml/Precision.h:19-84).

Every kernel reads and writes the engine's storage type (bf16 on a bf16 engine) unless this table says otherwise:
`Fp32` kernels always work on fp32 buffers, `Mixed` kernels take both (fp32 master / moment state beside bf16
parameters, casts, fp32 loss rows from bf16 logits).  Arithmetic inside every kernel is fp32 either way.
"""
from __future__ import annotations

import enum

from ..core.types import OaPrecision


class OaPrecisionTag(enum.IntEnum):
    Bf16 = 0
    Fp32 = 1
    Mixed = 2


# Kernels that are NOT plain storage-typed.  Names are the kernel registry's.
kPrecisionTable = {
    "adam_bf16_vec4_kernel": OaPrecisionTag.Mixed,        # bf16 parameters and gradients, fp32 masters and moments
    "adam_f32_kernel": OaPrecisionTag.Fp32,
    "dp_reduce_adam_gather_kernel": OaPrecisionTag.Mixed,  # bf16 peer gradients, fp32 sum and master shard, bf16 all-gather
    "cast_kernel": OaPrecisionTag.Mixed,
    "xent_kernel": OaPrecisionTag.Mixed,                  # bf16 logits in place, fp32 per-row loss
    "splitk_reduce_kernel": OaPrecisionTag.Mixed,         # fp32 partials to the output type
    "gemm_f32_kernel": OaPrecisionTag.Fp32,
    "attn_f32_kernel": OaPrecisionTag.Fp32,
    "mamba3_scan_fwd_kernel": OaPrecisionTag.Mixed,       # bf16 activations, fp32 state
    "mamba3_scan_bwd_kernel": OaPrecisionTag.Mixed,
    "clip_grad_norm_kernel": OaPrecisionTag.Mixed,
    "philox_uniform_kernel": OaPrecisionTag.Fp32,
    # names of the reference's own table, kept so that a lookup by its shader names answers the same
    "AdamwMixed": OaPrecisionTag.Mixed,
    "CastF32Bf16": OaPrecisionTag.Mixed,
}


def OaLookupPrecision(name: str) -> OaPrecisionTag:
    return kPrecisionTable.get(name, OaPrecisionTag.Bf16)


def OaPrecisionDtype(tag: OaPrecisionTag, engine_precision: OaPrecision) -> int:
    """Storage selector of a kernel: 1 = bf16, 0 = fp32."""
    if engine_precision != OaPrecision.BF16:
        return 0
    return 1 if tag == OaPrecisionTag.Bf16 else 0


def OaLoadStoreStrideBytes(tag: OaPrecisionTag, engine_precision: OaPrecision) -> int:
    return 2 if OaPrecisionDtype(tag, engine_precision) == 1 else 4


def OaPipelineNameIsF32Variant(name: str) -> bool:
    return len(name) >= 4 and name.endswith("_f32")
