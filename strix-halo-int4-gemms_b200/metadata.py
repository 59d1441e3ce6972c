"""Registry key schema: operand types, scale modes, epilogues, layouts, tile records.

Mirrors the names and values of the reference's ``metadata.py`` (enums at :19-60, ``ScaleSpec``
:63, ``TileConfig`` :84, ``KernelMetadata`` :110, ``make_kernel_id`` :150) so that code written
against the reference keeps working; what the fields *mean* is re-keyed to the sm_100a kernels:

* ``ARCH`` is ``"sm_100a"``;
* ``KernelSchedule`` names the launch form, which is what distinguishes one entry's launch from
  another's: ``STANDARD`` is the library's own choice for the shape (persistent grid; a CTA pair
  per 256-row tile when that pays, else one CTA per 128-row tile), ``PERSISTENT`` forces one CTA
  per tile on a persistent grid, ``PERSISTENT_2CTA`` forces CTA pairs (``tcgen05 cta_group::2``),
  ``TILE_PER_CTA`` launches one CTA per output tile like a plain non-persistent kernel;
* ``TileConfig.block_m / block_n`` are the rows and columns an entry's shapes must be multiples
  of: the output tile of the forced forms (128 or 256 rows, 256 columns, 128 for SwiGLU), and for
  ``STANDARD`` entries also the smaller row multiples the kernel accepts by masking a partial
  tile; ``block_k`` is the K multiple (32, the K of one ``tcgen05.mma kind::i8``);
* ``group_size_m`` is the raster width in row tiles passed to the launch (0: the library's default
  for the form), ``split_k`` the number of K slices (a real split with a second reduction kernel),
  ``num_warps`` the CTA size in warps, ``num_stages`` the depth of the shared-memory operand
  pipeline of the single-CTA form; ``waves_per_eu`` is kept for signature compatibility and always 0.
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Any

ARCH = "sm_100a"
ACC_DTYPE = "int32"
SCALE_DTYPE_BF16 = "bfloat16"
OUTPUT_DTYPE_BF16 = "bfloat16"
OUTPUT_DTYPE_FLOAT32 = "float32"
SUPPORTED_SUBCHANNELS = (32, 64, 128, 256)
SUPPORTED_SPLIT_K = (1, 2, 4, 8)
# b_scale for subchannel kernels is laid out (K-groups, output columns): one contiguous
# vector of column scales per K-group, next to the weight rows it scales.
RHS_SUBCHANNEL_SCALE_LAYOUT = "kgroup_output"


class OperandDType(str, enum.Enum):
    INT4 = "int4"
    INT8 = "int8"


class ScaleMode(str, enum.Enum):
    PER_CHANNEL = "per_channel"
    SUBCHANNEL = "subchannel"


class Epilogue(str, enum.Enum):
    NONE = "none"
    RELU2 = "relu2"
    SWIGLU = "swiglu"


class GemmLayout(str, enum.Enum):
    """First letter: A, second letter: B.  N = used as stored, T = stored transposed."""

    NN = "nn"
    NT = "nt"
    TN = "tn"
    TT = "tt"


SUPPORTED_GEMM_LAYOUTS = (GemmLayout.NN, GemmLayout.NT, GemmLayout.TN)


class KernelSchedule(str, enum.Enum):
    STANDARD = "standard"
    PERSISTENT = "persistent"
    PERSISTENT_2CTA = "persistent_2cta"
    TILE_PER_CTA = "tile_per_cta"


class KernelStatus(str, enum.Enum):
    PLANNED = "planned"
    GENERATED = "generated"
    COMPILED = "compiled"
    BENCHMARKED = "benchmarked"


@dataclasses.dataclass(frozen=True, slots=True)
class ScaleSpec:
    mode: ScaleMode
    subchannel_size: int | None = None

    def __post_init__(self) -> None:
        if self.mode is ScaleMode.PER_CHANNEL:
            if self.subchannel_size is not None:
                raise ValueError("per-channel scales must not set subchannel_size")
            return
        if self.subchannel_size not in SUPPORTED_SUBCHANNELS:
            raise ValueError(
                f"subchannel_size must be one of {SUPPORTED_SUBCHANNELS}; got {self.subchannel_size}"
            )

    @property
    def label(self) -> str:
        return "pc" if self.mode is ScaleMode.PER_CHANNEL else f"sc{self.subchannel_size}"


@dataclasses.dataclass(frozen=True, slots=True)
class TileConfig:
    block_m: int
    block_n: int
    block_k: int
    group_size_m: int
    num_warps: int
    num_stages: int
    waves_per_eu: int
    even_k: bool
    split_k: int = 1

    def __post_init__(self) -> None:
        if self.split_k not in SUPPORTED_SPLIT_K:
            raise ValueError(f"split_k must be one of {SUPPORTED_SPLIT_K}; got {self.split_k}")

    @property
    def label(self) -> str:
        parts = (
            f"bm{self.block_m}",
            f"bn{self.block_n}",
            f"bk{self.block_k}",
            f"gm{self.group_size_m}",
            f"w{self.num_warps}",
            f"s{self.num_stages}",
            f"weu{self.waves_per_eu}",
            f"sk{self.split_k}",
            "evenk" if self.even_k else "maskk",
        )
        return "_".join(parts)


def output_dtype_for_split_k(split_k: int) -> str:
    """Split-K variants hand back float32 partial-free sums; everything else stores bf16."""
    return OUTPUT_DTYPE_BF16 if split_k == 1 else OUTPUT_DTYPE_FLOAT32


@dataclasses.dataclass(frozen=True, slots=True)
class KernelMetadata:
    kernel_id: str
    arch: str
    a_dtype: OperandDType
    b_dtype: OperandDType
    acc_dtype: str
    output_dtype: str
    scale_dtype: str
    scale: ScaleSpec
    epilogue: Epilogue
    tile: TileConfig
    device_kernel: str
    layout: GemmLayout = GemmLayout.NN
    schedule: KernelSchedule = KernelSchedule.STANDARD
    status: KernelStatus = KernelStatus.COMPILED
    measured_tops: float | None = None
    notes: str = ""

    def to_dict(self) -> dict[str, Any]:
        out = dataclasses.asdict(self)
        out.update(
            a_dtype=self.a_dtype.value,
            b_dtype=self.b_dtype.value,
            scale={"mode": self.scale.mode.value, "subchannel_size": self.scale.subchannel_size},
            epilogue=self.epilogue.value,
            layout=self.layout.value,
            schedule=self.schedule.value,
            status=self.status.value,
            rhs_subchannel_scale_layout=(
                RHS_SUBCHANNEL_SCALE_LAYOUT if self.scale.mode is ScaleMode.SUBCHANNEL else None
            ),
        )
        return out


def make_kernel_id(
    dtype: OperandDType,
    scale: ScaleSpec,
    epilogue: Epilogue,
    tile: TileConfig,
    *,
    arch: str = ARCH,
    layout: GemmLayout = GemmLayout.NN,
    schedule: KernelSchedule = KernelSchedule.STANDARD,
) -> str:
    """``<arch>_<dt>x<dt>_<layout>_<scale>_<epilogue>[_<schedule>]_<tile label>``."""
    fields = [arch, f"{dtype.value}x{dtype.value}", layout.value, scale.label, epilogue.value]
    if schedule is not KernelSchedule.STANDARD:
        fields.append(schedule.value)
    fields.append(tile.label)
    return "_".join(fields)


def supported_scale_specs() -> tuple[ScaleSpec, ...]:
    subchannel = tuple(ScaleSpec(ScaleMode.SUBCHANNEL, size) for size in SUPPORTED_SUBCHANNELS)
    return subchannel + (ScaleSpec(ScaleMode.PER_CHANNEL),)
