"""The built library loads, exports every symbol include/conductor_b200.h declares, and its
struct layouts agree with what a C compiler makes of the header.  No compute calls: CPU only."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

from conductor_b200.codegen import kernel_templates as kt
from conductor_b200.compiler import loader

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "conductor_b200.h"


def declared_functions():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"CDR_API\s+[\w\s\*]+?\b(cdr_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("cdr_abi_version", "cdr_launch", "cdr_execute_host", "cdr_workspace_bytes", "cdr_status_string",
                 "cdr_last_error", "cdr_device_count", "cdr_device_status", "cdr_release_host_arena"):
        assert must in names


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(str(built_library))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(declared_functions()) == set(loader.SYMBOLS), "loader.SYMBOLS and the header disagree"


def test_loader_binds_and_checks_abi_version(built_library):
    lib = loader.load_library()
    assert lib.cdr_abi_version() == loader.ABI_VERSION
    assert lib.cdr_status_string(0) == b"ok"
    assert b"unsupported" in lib.cdr_status_string(-2)
    assert lib.cdr_last_error() is not None


def test_argument_errors_need_no_gpu(built_library):
    lib = loader.load_library()
    n = ctypes.c_size_t(7)
    # unknown template -> UNSUPPORTED before any CUDA call
    assert lib.cdr_workspace_bytes(99, None, 0, None, 0, None, 0, ctypes.byref(n)) == -2
    assert b"unknown template" in lib.cdr_last_error()
    # wrong parameter block size -> BAD_ARG
    p = kt.CdrGemmParams(0, 0)
    assert lib.cdr_workspace_bytes(1, None, 0, None, 0, ctypes.cast(ctypes.byref(p), ctypes.c_void_p),
                                   ctypes.sizeof(p), ctypes.byref(n)) == -1
    assert lib.cdr_workspace_bytes(1, None, 0, None, 0, None, 0, None) == -1


def test_generated_elementwise_source_compiles_without_a_gpu(built_library):
    """The run-time instance of an elementwise program: generated source is specialised with the
    program and the dtypes, and NVRTC accepts it for sm_100a (no device needed to compile)."""
    import torch

    import abi_util as abi
    from conductor_b200.codegen.operator_registry import EwOp
    from conductor_b200.compiler.executor import make_descriptors

    lib = loader.load_library()
    x, w, col = torch.zeros(8, 16), torch.zeros(16, dtype=torch.bfloat16), torch.zeros(8, 1, dtype=torch.float16)
    out = torch.zeros(8, 16, dtype=torch.bfloat16)
    prog = abi.ew_program(3, [
        (EwOp.MUL, 0, 1, 0, 0, torch.float32), (EwOp.TANH, 3, 0, 0, 0, torch.float32),
        (EwOp.ADDCMUL, 4, 2, 0, 0.5, torch.float32), (EwOp.RSUB_IMM, 5, 0, 0, 2.0, torch.bfloat16)],
        [6], [abi.FULL, abi.ROW, abi.COL])
    pp, ps = ctypes.cast(ctypes.byref(prog), ctypes.c_void_p), ctypes.sizeof(prog)
    buf = ctypes.create_string_buffer(1 << 16)
    ind, outd = make_descriptors([x, w, col]), make_descriptors([out])
    rc = lib.cdr_template_source(1, ind, 3, outd, 1, pp, ps, buf, len(buf), 0)
    assert rc == 0, lib.cdr_last_error()
    src = buf.value.decode()
    assert "cdr_jit_k" in src and "tanhf" in src and "un_bf16" in src and "% a.cols" in src
    # compile when NVRTC is installed; the library reports its absence as "unsupported"
    rc = lib.cdr_template_source(1, ind, 3, outd, 1, pp, ps, buf, len(buf), 1)
    if rc != 0:
        assert rc == -2 and b"NVRTC" in lib.cdr_last_error()
        if b"not available" not in lib.cdr_last_error():
            pytest.fail(lib.cdr_last_error().decode())
    # truncation keeps the terminator; integer programs have no run-time instance
    small = ctypes.create_string_buffer(32)
    assert lib.cdr_template_source(1, ind, 3, outd, 1, pp, ps, small, len(small), 0) == 0
    assert len(small.value) == 31
    xi = torch.zeros(8, 16, dtype=torch.int32)
    iprog = abi.ew_program(1, [(EwOp.ADD, 0, 0, 0, 0, torch.int32)], [1])
    assert lib.cdr_template_source(1, make_descriptors([xi]), 1, make_descriptors([xi]), 1,
                                      ctypes.cast(ctypes.byref(iprog), ctypes.c_void_p), ctypes.sizeof(iprog),
                                      buf, len(buf), 0) == -2
    assert lib.cdr_template_source(1, ind, 3, outd, 1, pp, ps, None, 0, 0) == -1
    assert lib.cdr_template_source(5, ind, 3, outd, 1, pp, ps, buf, len(buf), 0) == -2
    # an all-bf16 chain of exactly-rounding ops is emitted on bf16x2 instructions
    xb, wb = torch.zeros(8, 16, dtype=torch.bfloat16), torch.zeros(16, dtype=torch.bfloat16)
    pprog = abi.ew_program(2, [(EwOp.MUL, 0, 1, 0, 0, torch.bfloat16), (EwOp.RELU, 2, 0, 0, 0, torch.bfloat16),
                               (EwOp.ADD_IMM, 3, 0, 0, 1.5, torch.bfloat16)], [4], [abi.FULL, abi.ROW])
    args = (make_descriptors([xb, wb]), 2, make_descriptors([xb]), 1, ctypes.cast(ctypes.byref(pprog), ctypes.c_void_p),
            ctypes.sizeof(pprog), buf, len(buf))
    rc = lib.cdr_template_source(1, *args, 1)
    assert rc == 0 or b"not available" in lib.cdr_last_error(), lib.cdr_last_error()
    assert "= bmul(r0, r1)" in buf.value.decode() and "0x3fc03fc0u" in buf.value.decode()
    pprog.instr[2].imm = 0.1     # not a bf16 value: eager adds the fp32 constant, so no packed form
    assert lib.cdr_template_source(1, *args, 0) == 0 and "= bmul(r0, r1)" not in buf.value.decode()
    # chain + reduction over the last dimension: warp-per-row and CTA-per-row skeletons, every reduce op
    for cols in (64, 4096):
        for op in (1, 2, 3, 4):
            xr, wr = torch.zeros(4, cols, dtype=torch.bfloat16), torch.zeros(cols)
            rp = kt.CdrReduceParams()
            rp.chain = abi.ew_program(2, [(EwOp.MUL, 0, 1, 0, 0, torch.float32), (EwOp.EXP, 2, 0, 0, 0, torch.float32)],
                                      [3], [abi.FULL, abi.ROW])
            rp.reduce_op = op
            rc = lib.cdr_template_source(2, make_descriptors([xr, wr]), 2, make_descriptors([torch.zeros(4)]), 1,
                                         ctypes.cast(ctypes.byref(rp), ctypes.c_void_p), ctypes.sizeof(rp), buf, len(buf), 1)
            assert rc == 0 or b"not available" in lib.cdr_last_error(), lib.cdr_last_error()
            assert ("G = 256" if cols == 4096 else "G = 32") in buf.value.decode()
            # the same chain reduced over every element: persistent grid + ticket fold
            rc = lib.cdr_template_source(7, make_descriptors([xr, wr]), 2, make_descriptors([torch.zeros(1)]), 1,
                                         ctypes.cast(ctypes.byref(rp), ctypes.c_void_p), ctypes.sizeof(rp), buf, len(buf), 1)
            assert rc == 0 or b"not available" in lib.cdr_last_error(), lib.cdr_last_error()
            assert "atomicAdd(ticket" in buf.value.decode()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from conductor_b200.utils.exceptions import DeviceError

    monkeypatch.setenv("CONDUCTOR_B200_LIB", str(tmp_path / "nope.so"))
    loader.unload_library()
    try:
        with pytest.raises(DeviceError):
            loader.load_library()
    finally:
        monkeypatch.delenv("CONDUCTOR_B200_LIB")
        loader.unload_library()
        loader.load_library()


def test_struct_layouts_match_the_c_compiler(tmp_path):
    src = tmp_path / "sizes.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "conductor_b200.h"\n'
        "int main(void){printf(\"%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n\", sizeof(cdr_tensor), sizeof(cdr_ew_instr),"
        " sizeof(cdr_ew_params), sizeof(cdr_reduce_params), sizeof(cdr_gemm_params), sizeof(cdr_attn_params),"
        " offsetof(cdr_tensor, shape), offsetof(cdr_ew_params, instr), offsetof(cdr_reduce_params, reduce_op),"
        " sizeof(cdr_norm_params), offsetof(cdr_gemm_params, x_layout), sizeof(cdr_launch_item),"
        " offsetof(cdr_launch_item, inputs), offsetof(cdr_launch_item, workspace_bytes));"
        "return 0;}\n")
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c99", "-I", str(HEADER.parent), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [ctypes.sizeof(kt.CdrTensor), ctypes.sizeof(kt.CdrEwInstr), ctypes.sizeof(kt.CdrEwParams),
            ctypes.sizeof(kt.CdrReduceParams), ctypes.sizeof(kt.CdrGemmParams), ctypes.sizeof(kt.CdrAttnParams),
            kt.CdrTensor.shape.offset, kt.CdrEwParams.instr.offset, kt.CdrReduceParams.reduce_op.offset,
            ctypes.sizeof(kt.CdrNormParams), kt.CdrGemmParams.x_layout.offset, ctypes.sizeof(kt.CdrLaunchItem),
            kt.CdrLaunchItem.inputs.offset, kt.CdrLaunchItem.workspace_bytes.offset]
    assert got == want


def test_backend_registration_and_aliases():
    import torch

    import conductor

    assert "gcu" in torch._dynamo.list_backends(None)
    assert conductor.get_gcu_backend() is conductor.get_gcu_backend()
    assert isinstance(conductor.get_gcu_backend(), conductor.GCUBackend)
    assert conductor.register_gcu_backend() is True
    from conductor.utils.exceptions import CompilationError, ConductorError, ExecutionError  # noqa: F401
    import conductor_b200.utils.exceptions as impl

    assert ExecutionError is impl.ExecutionError and issubclass(CompilationError, ConductorError)
    assert conductor.get_config().runtime.device == "gcu"


def test_cpu_only_call_raises_device_error_not_fallback():
    """Without a CUDA device the compiled callable must refuse to run (no CPU path)."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import conductor  # noqa: F401
    from conductor.utils.exceptions import DeviceError

    torch._dynamo.reset()
    fn = torch.compile(lambda a, b, c: a * b + c, backend="gcu")
    with pytest.raises(Exception) as info:
        fn(torch.randn(4, 4), torch.randn(4, 4), torch.randn(4, 4))
    assert "DeviceError" in repr(info.value) or isinstance(info.value, DeviceError) or "no CUDA device" in str(info.value)
    torch._dynamo.reset()
