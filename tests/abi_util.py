"""Hand-built C-ABI calls for tests: no FX graph, no plan -- just ctypes structs and
``cdr_launch`` / ``cdr_execute_host``, the way a foreign-language binding would call them."""
import ctypes

import torch

from conductor_b200.codegen.kernel_templates import (
    CdrAttnParams, CdrEwInstr, CdrEwParams, CdrGemmParams, CdrReduceParams, CdrTensor)
from conductor_b200.codegen.operator_registry import EwOp, ReduceOp, Template
from conductor_b200.compiler.executor import make_descriptors
from conductor_b200.compiler.loader import load_library
from conductor_b200.utils.type_mapping import to_cdr_dtype

FULL, ROW, COL, SCALAR = range(4)


def ew_program(n_inputs, instrs, out_regs, modes=None):
    """instrs: list of (op, a, b, c, imm, torch_dtype)."""
    p = CdrEwParams()
    p.n_inputs, p.n_instr, p.n_outputs = n_inputs, len(instrs), len(out_regs)
    for i, m in enumerate(modes or [FULL] * n_inputs):
        p.input_mode[i] = m
    for i, r in enumerate(out_regs):
        p.out_reg[i] = r
    for i, (op, a, b, c, imm, dt) in enumerate(instrs):
        p.instr[i] = CdrEwInstr(op, a, b, c, float(imm), to_cdr_dtype(dt))
    return p


def mul_add_program(dtype=torch.float32, modes=None):
    return ew_program(3, [(EwOp.MUL, 0, 1, 0, 0, dtype), (EwOp.ADD, 3, 2, 0, 0, dtype)], [4], modes)


def launch(template, inputs, outputs, params=None, workspace=None, check=True):
    """cdr_launch on the current stream; returns the status."""
    lib = load_library()
    ind, outd = make_descriptors(inputs), make_descriptors(outputs)
    pp = ctypes.cast(ctypes.byref(params), ctypes.c_void_p) if params is not None else None
    ps = ctypes.sizeof(params) if params is not None else 0
    dev = (list(inputs) + list(outputs))[0].device
    stream = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        rc = lib.cdr_launch(template, ind, len(inputs), outd, len(outputs), pp, ps,
                            workspace.data_ptr() if workspace is not None else None,
                            workspace.numel() if workspace is not None else 0, stream)
    if check:
        assert rc == 0, (rc, lib.cdr_last_error().decode())
    return rc


def workspace_bytes(template, inputs, outputs, params=None):
    lib = load_library()
    ind, outd = make_descriptors(inputs), make_descriptors(outputs)
    pp = ctypes.cast(ctypes.byref(params), ctypes.c_void_p) if params is not None else None
    ps = ctypes.sizeof(params) if params is not None else 0
    n = ctypes.c_size_t(0)
    rc = lib.cdr_workspace_bytes(template, ind, len(inputs), outd, len(outputs), pp, ps, ctypes.byref(n))
    assert rc == 0, (rc, lib.cdr_last_error().decode())
    return n.value


def execute_host(template, inputs, outputs, params=None, device=0):
    lib = load_library()
    ind, outd = make_descriptors(inputs), make_descriptors(outputs)
    pp = ctypes.cast(ctypes.byref(params), ctypes.c_void_p) if params is not None else None
    ps = ctypes.sizeof(params) if params is not None else 0
    return lib.cdr_execute_host(template, ind, len(inputs), outd, len(outputs), pp, ps, device)
