"""Tracing JIT for elementwise chains: trace -> IR -> CSE / DCE -> one fused CUDA kernel
compiled with NVRTC for sm_100a (CPU tensors run the same IR through an interpreter).

Reference counterparts: cg_jit_begin_trace / cg_jit_end_trace, cg_ir_dce, cg_ir_cse,
cg_ir_fuse_ops, cg_jit_codegen_cuda, cg_jit_compile (include/cg_jit.h:150-238,
src/jit/graph_capture.c: the CUDA generator emits ADD/MUL/RELU/GELU only and nothing compiles
or runs it; cg_jit_execute is declared only).  The opcode set and names are those of
cg_ir_opcode; the host library (csrc/capi/jit*.cpp) carries the same passes for the C API.

    fused = fuse(lambda x, b: gelu(x + b) * 0.5)
    y = fused(x, bias)            # first call traces, generates, compiles; later calls launch

Inputs may be fp32 or bf16 and broadcast against the largest one along leading dimensions
(a [N] bias against [M, N], a scalar against anything); arithmetic is fp32; the result has the
first input's dtype.
"""
from __future__ import annotations

import ctypes
import hashlib
import math

import torch

UNARY = {"neg": "(-{a})", "exp": "expf({a})", "log": "logf({a})", "sqrt": "sqrtf({a})", "rsqrt": "rsqrtf({a})",
         "relu": "fmaxf({a}, 0.0f)", "sigmoid": "(1.0f / (1.0f + expf(-{a})))", "tanh": "tanhf({a})",
         "gelu": "(0.5f * {a} * (1.0f + tanhf(0.7978845608f * ({a} + 0.044715f * {a} * {a} * {a}))))"}
BINARY = {"add": "({a} + {b})", "sub": "({a} - {b})", "mul": "({a} * {b})", "div": "({a} / {b})"}
_TORCH = {"neg": torch.neg, "exp": torch.exp, "log": torch.log, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt, "relu": torch.relu,
          "sigmoid": torch.sigmoid, "tanh": torch.tanh, "gelu": lambda x: torch.nn.functional.gelu(x, approximate="tanh"),
          "add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div}


class Node:
    __slots__ = ("op", "inputs", "value", "id")

    def __init__(self, op, inputs=(), value=None):
        self.op, self.inputs, self.value, self.id = op, tuple(inputs), value, -1


class Var:
    """Symbolic value during tracing."""

    def __init__(self, graph, node):
        self.g, self.n = graph, node

    def _bin(self, op, other, swap=False):
        o = other if isinstance(other, Var) else self.g.const(float(other))
        a, b = (o, self) if swap else (self, o)
        return Var(self.g, self.g.add(Node(op, (a.n, b.n))))

    def __add__(self, o): return self._bin("add", o)
    def __radd__(self, o): return self._bin("add", o, True)
    def __sub__(self, o): return self._bin("sub", o)
    def __rsub__(self, o): return self._bin("sub", o, True)
    def __mul__(self, o): return self._bin("mul", o)
    def __rmul__(self, o): return self._bin("mul", o, True)
    def __truediv__(self, o): return self._bin("div", o)
    def __rtruediv__(self, o): return self._bin("div", o, True)
    def __neg__(self): return Var(self.g, self.g.add(Node("neg", (self.n,))))


def _unary(name):
    def f(x: Var) -> Var:
        return Var(x.g, x.g.add(Node(name, (x.n,))))
    f.__name__ = name
    return f


exp, log, sqrt, rsqrt, relu, sigmoid, tanh, gelu = (_unary(n) for n in ("exp", "log", "sqrt", "rsqrt", "relu", "sigmoid", "tanh", "gelu"))


class Graph:
    def __init__(self, n_inputs):
        self.nodes: list[Node] = []
        self.inputs = [self.add(Node("input", value=i)) for i in range(n_inputs)]
        self.output: Node | None = None

    def add(self, node):
        node.id = len(self.nodes)
        self.nodes.append(node)
        return node

    def const(self, v):
        return Var(self, self.add(Node("const", value=v)))

    # ---- passes
    def cse(self):
        seen, rename = {}, {}
        for n in self.nodes:
            n.inputs = tuple(rename.get(i.id, i) for i in n.inputs)
            ins = tuple(i.id for i in n.inputs)
            if n.op in ("add", "mul"):
                ins = tuple(sorted(ins))
            key = (n.op, ins, n.value)
            if n.op != "input" and key in seen:
                rename[n.id] = seen[key]
            else:
                seen[key] = n
        if self.output is not None:
            self.output = rename.get(self.output.id, self.output)

    def live(self):
        """Nodes reachable from the output, in program order (dead code elimination)."""
        keep, work = set(), [self.output]
        while work:
            n = work.pop()
            if n.id in keep:
                continue
            keep.add(n.id)
            work.extend(n.inputs)
        return [n for n in self.nodes if n.id in keep]

    # ---- code generation
    def cuda_source(self, in_dtypes, out_dtype, name="jit_kernel"):
        live = self.live()
        params, body = [], []
        for i, dt in enumerate(in_dtypes):
            params.append(f"const {dt}* __restrict__ in{i}, long mod{i}")
        params.append(f"{out_dtype}* __restrict__ out, long n")
        for n in live:
            v = f"v{n.id}"
            if n.op == "input":
                i = n.value
                load = f"in{i}[i % mod{i}]"
                body.append(f"    const float {v} = {'__bfloat162float(' + load + ')' if in_dtypes[i] == '__nv_bfloat16' else load};")
            elif n.op == "const":
                body.append(f"    const float {v} = {float(n.value)!r}f;")
            elif n.op in UNARY:
                body.append(f"    const float {v} = {UNARY[n.op].format(a='v%d' % n.inputs[0].id)};")
            else:
                body.append(f"    const float {v} = {BINARY[n.op].format(a='v%d' % n.inputs[0].id, b='v%d' % n.inputs[1].id)};")
        res = f"v{self.output.id}"
        store = f"__float2bfloat16({res})" if out_dtype == "__nv_bfloat16" else res
        return ("#include <cuda_bf16.h>\n"
                f"// fused elementwise: {sum(n.op not in ('input', 'const') for n in live)} ops\n"
                f"extern \"C\" __global__ void {name}({', '.join(params)}) {{\n"
                "  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {\n"
                + "\n".join(body) + f"\n    out[i] = {store};\n  }}\n}}\n")

    def interpret(self, tensors):
        vals = {}
        for n in self.live():
            if n.op == "input":
                vals[n.id] = tensors[n.value].float()
            elif n.op == "const":
                vals[n.id] = torch.tensor(n.value, dtype=torch.float32, device=tensors[0].device)
            else:
                vals[n.id] = _TORCH[n.op](*[vals[i.id] for i in n.inputs])
        return vals[self.output.id]


# ------------------------------------------------------------------ NVRTC
_MODULES: dict[str, object] = {}


def _include_dirs():
    import os
    cands = [os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")]
    return [d for d in cands if os.path.isdir(d)]


def compile_cuda(source: str, name: str = "jit_kernel"):
    """NVRTC -> cubin for sm_100a -> CUfunction (cached by source hash)."""
    from cuda.bindings import driver, nvrtc
    key = hashlib.sha1(source.encode()).hexdigest()
    if key in _MODULES:
        return _MODULES[key]
    err, prog = nvrtc.nvrtcCreateProgram(source.encode(), b"jit.cu", 0, [], [])
    opts = [b"--gpu-architecture=sm_100a"] + [f"-I{d}".encode() for d in _include_dirs()]
    (err,) = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    if err != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        _, ln = nvrtc.nvrtcGetProgramLogSize(prog)
        log = b" " * ln
        nvrtc.nvrtcGetProgramLog(prog, log)
        raise RuntimeError("NVRTC failed:\n" + log.decode(errors="replace") + "\n" + source)
    _, size = nvrtc.nvrtcGetCUBINSize(prog)
    cubin = b" " * size
    nvrtc.nvrtcGetCUBIN(prog, cubin)
    torch.cuda.current_device()                                 # the primary context must exist
    err, module = driver.cuModuleLoadData(cubin)
    if err != driver.CUresult.CUDA_SUCCESS:
        raise RuntimeError(f"cuModuleLoadData: {err}")
    err, fn = driver.cuModuleGetFunction(module, name.encode())
    if err != driver.CUresult.CUDA_SUCCESS:
        raise RuntimeError(f"cuModuleGetFunction: {err}")
    _MODULES[key] = (module, fn)
    return _MODULES[key]


def cubin_for(source: str) -> bytes:
    """Compile only (works without a GPU): used by the build check and the CPU tests."""
    from cuda.bindings import nvrtc
    err, prog = nvrtc.nvrtcCreateProgram(source.encode(), b"jit.cu", 0, [], [])
    opts = [b"--gpu-architecture=sm_100a"] + [f"-I{d}".encode() for d in _include_dirs()]
    (err,) = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    if err != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        _, ln = nvrtc.nvrtcGetProgramLogSize(prog)
        log = b" " * ln
        nvrtc.nvrtcGetProgramLog(prog, log)
        raise RuntimeError("NVRTC failed:\n" + log.decode(errors="replace"))
    _, size = nvrtc.nvrtcGetCUBINSize(prog)
    cubin = b" " * size
    nvrtc.nvrtcGetCUBIN(prog, cubin)
    return cubin


class FusedFunction:
    def __init__(self, fn):
        self.fn = fn
        self._graphs: dict[int, Graph] = {}
        self._kernels: dict[tuple, tuple] = {}
        self.launches = 0

    def graph(self, n_inputs: int) -> Graph:
        g = self._graphs.get(n_inputs)
        if g is None:
            g = Graph(n_inputs)
            out = self.fn(*[Var(g, n) for n in g.inputs])
            if not isinstance(out, Var):
                raise TypeError("the traced function must return an expression of its inputs")
            g.output = out.n
            g.cse()
            self._graphs[n_inputs] = g
        return g

    def source(self, *tensors) -> str:
        dts = ["__nv_bfloat16" if t.dtype == torch.bfloat16 else "float" for t in tensors]
        return self.graph(len(tensors)).cuda_source(dts, dts[0])

    def __call__(self, *tensors):
        g = self.graph(len(tensors))
        shape = torch.broadcast_shapes(*[t.shape for t in tensors])
        n = math.prod(shape)
        for t in tensors:
            if t.dtype not in (torch.float32, torch.bfloat16):
                raise TypeError("inputs must be float32 or bfloat16")
            k = t.numel()
            if n % max(k, 1) or tuple(t.shape) != tuple(shape[len(shape) - t.dim():]) and k != 1:
                raise ValueError("inputs must match the output shape or broadcast along leading dimensions")
        if not tensors[0].is_cuda:
            return g.interpret(list(tensors)).to(tensors[0].dtype).expand(shape).contiguous()
        from cuda.bindings import driver
        tensors = [t.contiguous() for t in tensors]
        dts = tuple("__nv_bfloat16" if t.dtype == torch.bfloat16 else "float" for t in tensors)
        key = (len(tensors), dts)
        if key not in self._kernels:
            self._kernels[key] = compile_cuda(g.cuda_source(list(dts), dts[0]))
        _, fn = self._kernels[key]
        out = torch.empty(shape, dtype=tensors[0].dtype, device=tensors[0].device)
        vals, types = [], []
        for t in tensors:
            vals += [t.data_ptr(), t.numel()]
            types += [ctypes.c_void_p, ctypes.c_long]
        vals += [out.data_ptr(), n]
        types += [ctypes.c_void_p, ctypes.c_long]
        threads = 256
        blocks = max(1, min((n + threads - 1) // threads, 148 * 8))
        (err,) = driver.cuLaunchKernel(fn, blocks, 1, 1, threads, 1, 1, 0, torch.cuda.current_stream().cuda_stream,
                                       (tuple(vals), tuple(types)), 0)
        if err != driver.CUresult.CUDA_SUCCESS:
            raise RuntimeError(f"cuLaunchKernel: {err}")
        self.launches += 1
        return out


def fuse(fn) -> FusedFunction:
    return FusedFunction(fn)
