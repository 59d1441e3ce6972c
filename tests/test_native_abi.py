"""The C ABI without a GPU: the library builds, loads, exports every symbol the header declares,
reports its status, and rejects bad arguments with rc=1 and a message (no kernel is launched).
Modelled on the reference's tests/test_native.py:34-180."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200_int4_gemms.h"


def _declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200_int4_gemms_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg, native_lib):
    from strix_halo_int4_gemms_b200 import native

    declared = _declared_symbols()
    assert len(declared) >= 12
    assert set(declared) == set(native.EXPORTED_SYMBOLS)
    lib = ctypes.CDLL(str(native_lib))
    for name in declared:
        assert hasattr(lib, name), name


def test_variant_record_matches_header(pkg):
    from strix_halo_int4_gemms_b200.native import DensePlan, GemmVariant

    plan = re.search(r"typedef struct b200_dense_plan \{(.*?)\}", HEADER.read_text(), flags=re.S).group(1)
    plan = re.sub(r"/\*.*?\*/", "", plan, flags=re.S)
    plan_fields = re.findall(r"int32_t\s+(\w+)(?:\[(\d+)\])?;", plan)
    assert [f[0] for f in plan_fields] == [name for name, _ in DensePlan._fields_]
    assert ctypes.sizeof(DensePlan) == 4 * sum(int(n or 1) for _, n in plan_fields) == 32

    body = re.search(r"typedef struct b200_gemm_variant \{(.*?)\}", HEADER.read_text(), flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"int32_t\s+(\w+)(?:\[(\d+)\])?;", body)
    assert [f[0] for f in fields] == [name for name, _ in GemmVariant._fields_]
    assert ctypes.sizeof(GemmVariant) == 4 * sum(int(n or 1) for _, n in fields) == 64


def test_runtime_status(pkg, native_lib):
    status = pkg.dispatch_runtime_status()
    assert status.library_path == native_lib and status.dispatch_version == 1
    assert status.has_compiled_code_objects is True
    assert status.has_cuda_runtime == torch.cuda.is_available()
    assert status.has_hip_runtime == status.has_cuda_runtime
    if not torch.cuda.is_available():
        assert status.has_linked_kernels is False
    with pytest.raises(RuntimeError, match="native dispatch library is not installed at"):
        pkg.dispatch_runtime_status("/nonexistent/libb200_int4_gemms.so")


def test_bad_arguments_fail_with_a_message(pkg, native_lib):
    from strix_halo_int4_gemms_b200 import native

    lib = native.load_dispatch_library()
    pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
    good = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=pc, epilogue=pkg.Epilogue.NONE, out_dtype=native.OUT_BF16)

    def dense(variant, ptrs=(0, 0, 0, 0, 0), shape=(128, 256, 64)):
        rc = lib.b200_int4_gemms_launch_dense(ctypes.byref(variant), 0, 0, *[ctypes.c_void_p(p) for p in ptrs], None, 0, *shape)
        return rc, lib.b200_int4_gemms_last_error().decode()

    assert dense(good) == (1, "a, b and c pointers must be non-null")
    assert dense(good, ptrs=(16, 16, 0, 0, 16)) == (1, "a_scale and b_scale pointers must be non-null")
    assert dense(good, ptrs=(16, 16, 16, 16, 16), shape=(0, 256, 64)) == (1, "m, n and k must be positive")
    bad = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=pc, epilogue=pkg.Epilogue.RELU2, out_dtype=native.OUT_F32, split_k=2)
    assert dense(bad, ptrs=(16, 16, 16, 16, 16)) == (1, "split_k > 1 needs epilogue NONE and float32 output")
    # the registry's launch forms map onto the variant record
    pair = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=pc, epilogue=pkg.Epilogue.NONE,
                               out_dtype=native.OUT_BF16, schedule=pkg.KernelSchedule.PERSISTENT_2CTA, group_m=8)
    assert (pair.schedule, pair.cta_group, pair.group_m) == (native.SCHEDULE_PERSISTENT, native.CTA_GROUP_PAIR, 8)
    assert (good.schedule, good.cta_group) == (native.SCHEDULE_PERSISTENT, native.CTA_GROUP_AUTO)
    plain = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=pc, epilogue=pkg.Epilogue.NONE,
                                out_dtype=native.OUT_BF16, schedule=pkg.KernelSchedule.TILE_PER_CTA)
    assert (plain.schedule, plain.cta_group) == (native.SCHEDULE_TILE_PER_CTA, native.CTA_GROUP_SINGLE)
    split = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=pc, epilogue=pkg.Epilogue.NONE, out_dtype=native.OUT_F32, split_k=4)
    need = lib.b200_int4_gemms_dense_workspace_bytes(ctypes.byref(split), 128, 256, 1024)
    assert need == 4 * 128 * 256 * 4
    assert lib.b200_int4_gemms_dense_workspace_bytes(ctypes.byref(split), 128, 256, 256) == 2 * 128 * 256 * 4   # two K blocks: two slices
    assert lib.b200_int4_gemms_dense_workspace_bytes(ctypes.byref(split), 128, 256, 64) == 0                    # one K block: no split
    assert lib.b200_int4_gemms_dense_workspace_bytes(ctypes.byref(good), 128, 256, 1024) == 0
    assert lib.b200_int4_gemms_last_launch_path() == native.LAUNCHED_NOTHING
    bad = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=pc, epilogue=pkg.Epilogue.NONE, out_dtype=native.OUT_BF16)
    bad.subchannel, bad.scale_mode = 48, 1
    assert dense(bad, ptrs=(16, 16, 16, 16, 16)) == (1, "variant.subchannel must be 32, 64, 128 or 256")
    rc = lib.b200_int4_gemms_launch_dense(None, 0, 0, None, None, None, None, None, None, 0, 1, 1, 1)
    assert rc == 1 and lib.b200_int4_gemms_last_error().decode() == "variant must be non-null"
    with pytest.raises(RuntimeError, match="a, b and c pointers must be non-null"):
        native.launch_dense(good, device_index=0, stream_handle=0, a_ptr=0, b_ptr=0, a_scale_ptr=0, b_scale_ptr=0, c_ptr=0, m=1, n=1, k=1)


def test_ragged_entry_points_check_arguments(pkg, native_lib):
    from strix_halo_int4_gemms_b200 import native

    lib = native.load_dispatch_library()
    pc = pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL)
    v8 = native.make_variant(dtype=pkg.OperandDType.INT8, layout=pkg.GemmLayout.NN, scale=pc, epilogue=pkg.Epilogue.NONE, out_dtype=native.OUT_BF16)
    nine = [ctypes.c_void_p(16)] * 9
    rc = lib.b200_int4_gemms_launch_ragged_fwd(ctypes.byref(v8), 0, 0, *nine, 128, 256, 32, 1, 1, 1, 128)
    assert rc == 1 and lib.b200_int4_gemms_last_error().decode() == "ragged kernels take packed int4 operands"
    v4 = native.make_variant(dtype=pkg.OperandDType.INT4, layout=pkg.GemmLayout.NN, scale=pc, epilogue=pkg.Epilogue.NONE, out_dtype=native.OUT_BF16)
    rc = lib.b200_int4_gemms_launch_ragged_fwd(ctypes.byref(v4), 0, 0, *([ctypes.c_void_p(0)] * 9), 128, 256, 32, 1, 1, 1, 128)
    assert rc == 1 and "pointers must be non-null" in lib.b200_int4_gemms_last_error().decode()
    rc = lib.b200_int4_gemms_launch_ragged_fwd(ctypes.byref(v4), 0, 0, *nine, 128, 256, 32, 1, 1, 1, 264)
    assert rc == 1 and lib.b200_int4_gemms_last_error().decode() == "block_rows must be in [1, 256]"
    rc = lib.b200_int4_gemms_launch_ragged_bwd(ctypes.byref(v4), 0, 0, *([ctypes.c_void_p(16)] * 6), 128, 256, 32, 1, 2)
    assert rc == 1 and lib.b200_int4_gemms_last_error().decode() == "ragged backward stores float32"


def test_launcher_validation_before_any_device_work(pkg):
    """Python-side checks of launch_generated_kernel that need no GPU (reference tests/test_native.py:131-157)."""
    from strix_halo_int4_gemms_b200.native import block_size, launch_grid

    k = pkg.default_registry.select(
        dtype=pkg.OperandDType.INT4, scale=pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL), epilogue=pkg.Epilogue.NONE, m=4096, n=4096, k=4096
    )
    assert block_size(k) == 448  # 2 + 4 + 8 warps: TMA, MMA, epilogue, unpack
    assert launch_grid(k, 4096, 4096) == (148, 1, 1)

    def form(schedule):
        return pkg.default_registry.select(
            dtype=pkg.OperandDType.INT4, scale=pkg.ScaleSpec(pkg.ScaleMode.PER_CHANNEL), epilogue=pkg.Epilogue.NONE,
            m=4096, n=4096, k=4096, schedule=schedule)

    assert launch_grid(form(pkg.KernelSchedule.PERSISTENT), 4096, 4096) == (148, 1, 1)
    assert launch_grid(form(pkg.KernelSchedule.PERSISTENT_2CTA), 4096, 4096) == (148, 1, 1)   # 74 pairs
    assert launch_grid(form(pkg.KernelSchedule.PERSISTENT_2CTA), 512, 512) == (8, 1, 1)       # 4 tiles of 256 x 256
    assert launch_grid(form(pkg.KernelSchedule.TILE_PER_CTA), 4096, 4096) == (512, 1, 1)
    a = torch.zeros((128, 32), dtype=torch.uint8)
    b = torch.zeros((32, 256), dtype=torch.uint8)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="require a CUDA torch device"):
            pkg.launch_generated_kernel(a, b, kernel=k, a_scale=torch.ones(128), b_scale=torch.ones(256))
