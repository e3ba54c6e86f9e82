"""Runs in a process of its own, because the reference and this library cannot both be ``LCT``.

    python tests/reference_runner.py bits    --out f.npz [--sizes RxC,RxC --steps S]
    python tests/reference_runner.py bench   --out f.json [--iters N] [--autotune]
    python tests/reference_runner.py dropin  --out f.json
    python tests/reference_runner.py interchange --out f.json

``bits`` and ``bench`` import the UNMODIFIED reference (a copy of its checkout under
``baseline/_ref``, made by ``__graft_entry__.build()`` where the checkout exists) with its Triton
kernels compiled for the GPU at hand: the configuration-4 recurrence through the reference's own
fused path, dumped step by step for the parity test, and the reference's kernels timed on
configurations 2 and 4 as the bar this library's kernels are measured against.

``interchange`` loads both codecs side by side and lets each decode what the other compressed
(through the reference's generic kernels and through its A100 decoder).

``dropin`` does the opposite: it installs THIS library under the name ``LCT``
(``compat.install_as_lct``), lets the reference's callers - ``examples/benchmarks`` and
``LCT/components/{layers,ops}.py`` - resolve on top of it unmodified, and runs their own checks.

TEST INFRASTRUCTURE: only ``tests/`` and ``bench.py`` start this script.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.path.join(ROOT, "baseline", "_ref")


def available() -> bool:
    return os.path.isdir(os.path.join(REFERENCE, "LCT"))


def _load_reference(autotune: bool):
    os.environ["LCT_REFERENCE_ROOT"] = REFERENCE
    os.environ["TRITON_INTERPRET"] = "0"          # the compiled kernels, not the interpreter
    # "5090": one launch configuration per kernel (no tuning runs); "": the reference's own
    # default lists, tuned on this GPU on first use.
    os.environ["LCT_REFERENCE_BACKEND"] = "" if autotune else "5090"
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import reference_shim  # noqa: F401
    _leave_out_warp_specialization()


def _leave_out_warp_specialization() -> None:
    """Triton 3.6 runs its automatic warp-specialisation pass on every kernel it compiles for
    compute capability 10.x, and that pass aborts on the reference's decoder
    (``LCT/kernels/generic/decode.py:291``: "Pipeline failed while executing
    TritonGPUAutomaticWarpSpecialization ... NVWSInsertAref").  The pass is an optimisation, so
    the reference's kernels are compiled without it here; the reference itself is untouched."""
    try:
        from triton._C.libtriton import passes

        passes.ttgpuir.add_warp_specialize = lambda pass_manager, num_stages: None
    except (ImportError, AttributeError):
        pass


def _sha(t) -> str:
    return hashlib.sha256(t.detach().contiguous().cpu().numpy().tobytes()).hexdigest()[:16]


def config4_inputs(rows: int, cols: int, steps: int):
    """Seeded inputs of the configuration-4 recurrence (CPU generator: the same on every machine)."""
    import torch

    g = torch.Generator().manual_seed(10)
    momentum = (torch.randn(rows, cols, generator=g) * 1e-3).to(torch.bfloat16)
    grads = []
    for step in range(steps):
        gs = torch.Generator().manual_seed(100 + step)
        grads.append((torch.randn(rows, cols, generator=gs) * 1e-3).to(torch.bfloat16))
    return momentum, grads


def mode_bits(args) -> None:
    import numpy as np
    import torch

    _load_reference(autotune=False)
    from LCT.LCTensor import LCTTensor
    from LCT.comp_format import Distribution, DistType, NoiseLevel
    from LCT.tensor_buffer import TensorBuffer

    buffer = TensorBuffer(64 << 20, device="cuda")
    dist = Distribution(DistType.GAUSSIAN, noise_level=NoiseLevel.MEDIUM)
    alpha = torch.tensor([0.95], dtype=torch.float32, device="cuda")
    out = {}
    for index, size in enumerate(args.sizes.split(",")):
        rows, cols = (int(v) for v in size.split("x"))
        momentum, grads = config4_inputs(rows, cols, args.steps)
        state = LCTTensor(momentum.cuda(), buffer, dist)
        for step, grad in enumerate(grads):
            state.mul_add_(alpha, grad.cuda())
            c = state.x
            dense = state.decompress()
            key = f"{size}_{step}"
            out["dense_sha_" + key] = np.array(_sha(dense.view(torch.int16)))
            out["side_sha_" + key] = np.array(_sha(c.sign_mantissa))
            out["center_" + key] = np.array(int(c.center.item()))
            out["count_" + key] = np.array(int(c.fallback_count.item()))
            out["used_" + key] = np.array(int(c.fallback_used.item()))
            out["memory_size_" + key] = np.array(int(c.memory_size()))
            out["decode_table_sha_" + key] = np.array(_sha(c.decode_table))
            if index == 0:   # the first (small) size also keeps the raw payload words
                out["payload_" + key] = c.data.cpu().numpy()
        state.free()
    torch.cuda.synchronize()
    np.savez(args.out, **out)


def _time(fn, iters: int, warmup: int = 5) -> float:
    import torch

    flush = _time.flush
    for _ in range(warmup):
        fn()
    spans = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        spans.append((a, b))
    torch.cuda.synchronize()
    times = sorted(a.elapsed_time(b) for a, b in spans)
    return times[len(times) // 2]


def mode_bench(args) -> None:
    import torch

    _load_reference(autotune=args.autotune)
    sys.path.insert(0, ROOT)
    sys.argv = sys.argv[:1]
    import bench  # the workload generator only (no import of this library's package)
    from LCT.LCTensor import LCTTensor
    from LCT.comp_format import Distribution, DistType, NoiseLevel
    from LCT.operations import compress, decompress
    from LCT.tensor_buffer import TensorBuffer

    _time.flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    buffer = TensorBuffer(64 << 20, device="cuda")
    out = {"autotune": bool(args.autotune), "triton": __import__("triton").__version__}
    # configuration 2
    x = bench.make_workload(1).cuda()
    dist = Distribution(DistType.LAPLACE, param=0.02)
    c = compress(x, dist, buffer)
    assert torch.equal(decompress(c).view(torch.int16), x.view(torch.int16))
    out["config2_memory_size"] = int(c.memory_size())
    keep = [c]

    def encode():
        keep.append(compress(x, dist, buffer))
        keep.pop(0).free()

    out["config2_compress_ms"] = _time(encode, args.iters)
    out["config2_decompress_ms"] = _time(lambda: decompress(keep[0]), args.iters)
    keep.pop().free()
    del x
    # configuration 4: one tensor-step of the fused update
    momentum, grads = config4_inputs(4096, 4096, 1)
    dist4 = Distribution(DistType.GAUSSIAN, noise_level=NoiseLevel.MEDIUM)
    state = LCTTensor(momentum.cuda(), buffer, dist4)
    grad = grads[0].cuda()
    alpha = torch.tensor([0.95], dtype=torch.float32, device="cuda")
    out["config4_mul_add_ms"] = _time(lambda: state.mul_add_(alpha, grad), args.iters)
    with open(args.out, "w") as handle:
        json.dump(out, handle)


def _serve_reference_components() -> None:
    """Modules of ``LCT.components`` that this library does not have (layers, ops, mlps, ...)
    resolve to the reference's files, byte for byte.  The reference targets Python 3.14, whose
    annotations are evaluated lazily; on older interpreters the files that annotate with
    TYPE_CHECKING-only names get ``from __future__ import annotations`` from the loader
    (``ops.py`` is left alone: its custom-op schemas are inferred from real annotation objects)."""
    import importlib.machinery

    import LCT.components as components

    directory = os.path.join(REFERENCE, "LCT", "components")
    future = "from __future__ import annotations"

    class Loader(importlib.machinery.SourceFileLoader):
        def source_to_code(self, data, path, *, _optimize=-1):
            text = data.decode() if isinstance(data, bytes) else data
            if sys.version_info < (3, 14) and not path.endswith("ops.py") and future not in text:
                stripped = text.lstrip()
                if stripped.startswith(('"""', "'''")):
                    quote = stripped[:3]
                    end = text.index(quote, text.index(quote) + 3) + 3
                    text = text[:end] + ";" + future + text[end:]
                else:
                    text = future + ";" + text
            return super().source_to_code(text, path, _optimize=_optimize)

    class Finder(importlib.machinery.PathFinder):
        @classmethod
        def find_spec(cls, name, path=None, target=None):
            if not name.startswith("LCT.components.") or name in sys.modules:
                return None
            spec = importlib.machinery.PathFinder.find_spec(name, [directory], target)
            if spec is not None and spec.origin and spec.origin.endswith(".py"):
                spec.loader = Loader(name, spec.origin)
            return spec

    components.__path__.append(directory)
    sys.meta_path.insert(0, Finder)


def mode_dropin(args) -> None:
    """The reference's callers, unmodified, on this library installed as ``LCT``."""
    import torch

    sys.path.insert(0, ROOT)
    import losslessly_compressed_tensors_b200.compat as compat

    compat.install_as_lct()
    _serve_reference_components()
    sys.path.insert(0, REFERENCE)   # for `examples.benchmarks`
    report = {}

    # 1. examples/benchmarks/benchmark_lct.py: its run_case (round trip + ratio ceiling, :108-157)
    import examples.benchmarks.benchmark_lct as codec_bench
    from LCT.tensor_buffer import TensorBuffer

    codec_bench.WARMUP, codec_bench.ITERS = 1, 2
    buffer = TensorBuffer(64 << 20, device="cuda")
    for name, max_ratio in codec_bench.CASES:
        codec_bench.run_case(name, args.elements, max_ratio, buffer)
    report["benchmark_lct_cases"] = len(codec_bench.CASES)

    # 2. examples/benchmarks/benchmark_pointwise.py: check_result (:35-44) on the expressions
    #    of its main() (:133-151), every fused operation, dense and compressed output.
    import examples.benchmarks.benchmark_pointwise as fused_bench
    from LCT.comp_format import Distribution, DistType
    from LCT.operations import (a_compA_add_B, a_compA_add_b_B, a_compA_add_compB, compA_add_B,
                                compA_mul_B, compress)

    n = args.elements
    dist = Distribution(DistType.GAUSSIAN, param=2.0)
    a = codec_bench.make_gaussian(n, std=dist.param, seed=0)
    b = codec_bench.make_gaussian(n, std=dist.param, seed=1)
    multiplier = codec_bench.make_gaussian(n, mean=1.0, std=0.01, seed=2)
    alpha = torch.tensor([-0.5], device="cuda", dtype=torch.float32)
    beta = torch.tensor([-0.02], device="cuda", dtype=torch.float32)
    a_comp, b_comp = compress(a, dist, buffer), compress(b, dist, buffer)
    references = {
        "compA_add_B": lambda s, e: a[s:e] + b[s:e],
        "compA_mul_B": lambda s, e: a[s:e] * multiplier[s:e],
        "a_compA_add_B": lambda s, e: (a[s:e].float() * alpha + b[s:e].float()).to(torch.bfloat16),
        "a_compA_add_compB": lambda s, e: (a[s:e].float() * alpha + b[s:e].float()).to(torch.bfloat16),
        "a_compA_add_b_B": lambda s, e: fused_bench.two_scale_add(a[s:e], b[s:e], alpha, beta),
    }
    checked = 0
    for dense in (True, False):
        kw = dict(dense_output=dense, buffer=buffer, distribution=dist)
        results = {
            "compA_add_B": compA_add_B(a_comp, b, **kw),
            "compA_mul_B": compA_mul_B(a_comp, multiplier, **kw),
            "a_compA_add_B": a_compA_add_B(a_comp, alpha, b, **kw),
            "a_compA_add_compB": a_compA_add_compB(a_comp, alpha, b_comp, **kw),
            "a_compA_add_b_B": a_compA_add_b_B(a_comp, alpha, b, beta, **kw),
        }
        for name, result in results.items():
            fused_bench.check_result(result, references[name], a.shape)
            fused_bench.release(result)
            checked += 1
    report["benchmark_pointwise_checks"] = checked

    # 3. LCT/components/layers.py: RMSLinear (:22-72) forward + backward with a compressed
    #    saved activation, against the same layer with the activation kept dense.
    from LCT.components.layers import RMSLinear
    import LCT.components.mlps  # noqa: F401  (imports cleanly on the drop-in as well)

    torch.manual_seed(0)
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    weight = (torch.randn(384, 512, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_()
    gain = torch.ones(512, device="cuda", dtype=torch.float32, requires_grad=True)
    bias = torch.zeros(384, device="cuda", dtype=torch.float32, requires_grad=True)
    grads = {}
    for compressed in (False, True):
        for t in (x, weight, gain, bias):
            t.grad = None
        y = RMSLinear.apply(x, weight, gain, bias, buffer, compressed, None, 1)
        y.float().square().mean().backward()
        grads[compressed] = [t.grad.clone() for t in (x, weight, gain, bias)] + [y.detach().clone()]
    for dense_value, compressed_value in zip(grads[False], grads[True]):
        assert torch.equal(dense_value, compressed_value), "RMSLinear: compressed activation changed a result"
    report["rms_linear"] = "forward and backward identical with the saved activation compressed"

    # 4. The other activation layers of the reference, same criterion (outputs and every gradient
    #    bit-identical with the saved activations compressed into the shared arena), and the arena
    #    empty afterwards: Relu2Linear (layers.py:182-227), the shared-input Q/K/V projection
    #    (rms_norm_qkv, :75-140), RMSNormFunction (:143-179), FFN and RMSFFN (mlps.py:41-150), whose
    #    saved tensors are LCTTensor wrappers.
    from LCT.components.layers import Relu2Linear, RMSNormFunction, rms_norm_qkv
    from LCT.components.mlps import FFN, RMSFFN
    from LCT.tensor_buffer import _free_regions_snapshot

    def bf16(*shape, scale=1.0, grad=True):
        return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16).requires_grad_(grad)

    def same_with_and_without(name, leaves, run):
        results = {}
        for compressed in (False, True):
            for t in leaves:
                t.grad = None
            outputs = run(compressed)
            outputs = outputs if isinstance(outputs, tuple) else (outputs,)
            sum(o.float().square().mean() for o in outputs).backward()
            results[compressed] = [t.grad.clone() for t in leaves] + [o.detach().clone() for o in outputs]
        for dense_value, compressed_value in zip(results[False], results[True]):
            assert torch.equal(dense_value, compressed_value), f"{name}: compressed activation changed a result"
        assert _free_regions_snapshot(buffer) == free_before, f"{name}: arena regions not returned"
        report[name] = "forward and backward identical with the saved activations compressed"

    for c in (a_comp, b_comp):
        c.free()
    free_before = _free_regions_snapshot(buffer)
    z, w2, b2 = bf16(512, 1024), bf16(256, 1024, scale=0.02), torch.zeros(256, device="cuda", requires_grad=True)
    same_with_and_without("relu2_linear", (z, w2, b2),
                          lambda c: Relu2Linear.apply(z, w2, b2, buffer, c, None, 1))
    xq = bf16(512, 256)
    gain_q = torch.ones(256, device="cuda", requires_grad=True)
    projections = [torch.nn.Linear(256, 128, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    leaves = [xq, gain_q] + [p for m in projections for p in (m.weight, m.bias)]
    same_with_and_without("rms_norm_qkv", leaves,
                          lambda c: rms_norm_qkv(xq, gain_q, *projections, buffer=buffer, compressed=c,
                                                 min_elements=1))
    xn, gains = bf16(512, 256), torch.ones(256, device="cuda", requires_grad=True)
    same_with_and_without("rms_norm_function", (xn, gains),
                          lambda c: RMSNormFunction.apply(xn, gains, buffer, c, None, 1))
    xf, w1f, w2f = bf16(512, 256), bf16(1024, 256, scale=0.05), bf16(256, 1024, scale=0.05)
    same_with_and_without("ffn", (xf, w1f, w2f), lambda c: FFN.apply(xf, w1f, w2f, buffer, c))
    if hasattr(torch.ops.aten, "_fused_rms_norm"):      # the operator RMSFFN is written on
        same_with_and_without("rms_ffn", (xf, w1f, w2f), lambda c: RMSFFN.apply(xf, w1f, w2f, buffer, c))
    else:
        report["rms_ffn"] = "not run: this PyTorch has no aten._fused_rms_norm"
    # FlashAttention (layers.py:253-305): Q, K, V and the attention output cached compressed
    # (BHTD views of contiguous BTHD storage, as its trainer supplies them).
    from LCT.components.layers import FlashAttention

    batch, length, heads, head_dim = 2, 256, 4, 64
    qkv = [(torch.randn(batch, length, heads, head_dim, device="cuda") * 0.5).to(torch.bfloat16)
           .requires_grad_() for _ in range(3)]
    w_o = bf16(128, heads * head_dim, scale=0.05)
    b_o = torch.zeros(128, device="cuda", requires_grad=True)
    try:
        same_with_and_without(
            "flash_attention", (*qkv, w_o, b_o),
            lambda c: FlashAttention.apply(*(t.transpose(1, 2) for t in qkv), w_o, b_o, buffer, c,
                                           None, 1))
    except (RuntimeError, NotImplementedError) as error:
        if "flash" not in str(error).lower():
            raise
        report["flash_attention"] = f"not run: {error}"[:200]   # no flash kernel for this GPU in this PyTorch
    # 5. The reference's own optimizers (LCT/components/sparse_utils.py, loaded from its file under
    #    another module name: this library has a module of that name too), unmodified, with their
    #    state compressed by this library: Muon and AdamW must follow their dense-state
    #    trajectories bit for bit (the codec is lossless), SGDM must run its fused updates.
    import importlib.util

    source_path = os.path.join(REFERENCE, "LCT", "components", "sparse_utils.py")
    with open(source_path) as handle:
        source = "from __future__ import annotations\n" + handle.read()
    spec = importlib.util.spec_from_loader("reference_sparse_utils", loader=None)
    reference_optimizers = importlib.util.module_from_spec(spec)
    reference_optimizers.__file__ = source_path
    exec(compile(source, source_path, "exec"), reference_optimizers.__dict__)
    from LCT.LCTensor import LCTTensor as OurWrapper

    shapes = [(256, 384), (384, 256), (128, 128)]

    def fresh(seed):
        gen = torch.Generator(device="cuda").manual_seed(seed)
        return [(torch.randn(shape, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
                for shape in shapes]

    def gradients(step):
        gen = torch.Generator(device="cuda").manual_seed(100 + step)
        return [(torch.randn(shape, device="cuda", generator=gen) * 0.01).to(torch.bfloat16)
                for shape in shapes]

    def make(kind, params, compressed):
        if kind == "muon":
            return reference_optimizers.SparseMuon(params, lr=0.02, weight_decay=0.01, buffer=buffer,
                                                   compressed=compressed, ns_iters=3)
        return reference_optimizers.SparseAdamW([dict(params=params, lr=1e-2)], weight_decay=0.1,
                                                compressed=compressed, buffer=buffer)

    for kind in ("muon", "adamw"):
        with_state, dense_state = fresh(7), fresh(7)
        opt_a, opt_b = make(kind, with_state, True), make(kind, dense_state, False)
        for step in range(3):
            for pa, pb, grad in zip(with_state, dense_state, gradients(step)):
                pa.grad, pb.grad = grad.clone(), grad.clone()
            opt_a.step()
            opt_b.step()
            for pa, pb in zip(with_state, dense_state):
                assert torch.equal(pa, pb), f"{kind}: parameters differ at step {step}"
        if kind == "muon":
            states = list(zip(opt_a.momentums, opt_b.momentums))
        else:
            states = [(opt_a.state[pa][key], opt_b.state[pb][key])
                      for pa, pb in zip(with_state, dense_state) for key in ("exp_avg", "exp_avg_sq")]
        for compressed_state, dense_value in states:
            assert isinstance(compressed_state, OurWrapper), f"{kind}: state is not compressed"
            assert torch.equal(compressed_state.decompress(), dense_value), f"{kind}: state differs"
            compressed_state.free()
        report["reference_" + kind] = "compressed-state trajectory identical to the dense-state one"
    params = fresh(8)
    sgdm = reference_optimizers.SparseSGDM(params, lr=0.1, momentum=0.9, buffer=buffer, compressed=True)
    for step in range(3):
        for p, grad in zip(params, gradients(step)):
            p.grad = grad
        sgdm.step()
    assert all(torch.isfinite(p.float()).all() for p in params)
    for state in sgdm.momentums:
        state.free()
    assert _free_regions_snapshot(buffer) == free_before, "optimizers: arena regions not returned"
    report["reference_sgdm"] = "three fused steps"
    torch.cuda.synchronize()
    with open(args.out, "w") as handle:
        json.dump(report, handle)


def mode_interchange(args) -> None:
    """Both codecs in one process (the reference as ``LCT``, this library under its own name):
    what one compresses the other must decode, for private and arena-held overflow, all layouts,
    ragged sizes - through the reference's generic kernels and through its A100 decoder, whose
    docstring promises the same payload (``LCT/kernels/a100/decode.py:13-15``)."""
    import dataclasses

    import torch

    _load_reference(autotune=False)
    import LCT.kernels.backends as ref_backends
    import LCT.kernels.dispatch as ref_dispatch
    from LCT import comp_format as rf, operations as ref_ops
    from LCT.comp_tensor import CompressedTensor as RefTensor
    from LCT.tensor_buffer import TensorBuffer as RefBuffer

    sys.path.insert(0, ROOT)
    from losslessly_compressed_tensors_b200 import comp_format as of, operations as our_ops
    from losslessly_compressed_tensors_b200.comp_tensor import CompressedTensor as OurTensor
    from losslessly_compressed_tensors_b200.tensor_buffer import TensorBuffer as OurBuffer

    def translate(c, target_cls, fmt):
        """The same fields under the other library's types (tensors are shared, not copied)."""
        values = {}
        for f in dataclasses.fields(target_cls):
            v = getattr(c, f.name)
            if f.name == "distribution":
                v = fmt.Distribution(fmt.DistType[v.family.name], param=v.param, mean=v.mean,
                                     zero_prob=v.zero_prob, noise_level=fmt.NoiseLevel[v.noise_level.name])
            elif f.name == "layout":
                v = fmt.StorageLayout[v.name]
            elif f.name == "buffer":
                v = None                     # only free() uses it
            values[f.name] = v
        return target_cls(**values)

    g = torch.Generator().manual_seed(11)

    def tensor(shape, kind):
        x = torch.randn(shape, generator=g)
        if kind == "heavy":                  # a wide spread of exponents: overflow lanes
            x = x * torch.exp(torch.randn(shape, generator=g) * 4)
        elif kind == "relu":
            x = x.relu()
        else:
            x = x * 0.02
        return x.to(torch.bfloat16).cuda()

    cases = [("laplace-clean", dict(family="LAPLACE", param=0.02), "plain", (1024, 1024)),
             ("laplace-clean-overflow", dict(family="LAPLACE", param=0.02), "heavy", (1000, 777)),
             ("gaussian-clean", dict(family="GAUSSIAN"), "heavy", (300, 700)),
             ("gaussian-medium", dict(family="GAUSSIAN", noise_level="MEDIUM"), "plain", (2048, 512)),
             ("sparse-relu", dict(family="LAPLACE", zero_prob=0.5, noise_level="SPARSE"), "relu", (512, 4096)),
             ("empirical-high", dict(family="EMPIRICAL", noise_level="HIGH"), "heavy", (65537,))]

    def dist_of(fmt, spec):
        return fmt.Distribution(fmt.DistType[spec["family"]], param=spec.get("param", 1.0),
                                zero_prob=spec.get("zero_prob", 0.0),
                                noise_level=fmt.NoiseLevel[spec.get("noise_level", "CLEAN")])

    report = {"cases": {}}
    stock = ref_dispatch.backend_for
    for backend in ("generic", "a100"):
        if backend == "a100":
            try:
                a100 = ref_backends._a100_backend()
            except Exception as error:          # the backend does not build here: say so, go on
                report["a100"] = f"unavailable: {type(error).__name__}: {error}"[:300]
                break
            ref_dispatch.backend_for = lambda device: a100
        try:
            for name, spec, kind, shape in cases:
                x = tensor(shape, kind)
                for buffered in (False, True):
                    ours = our_ops.compress(x, dist_of(of, spec), OurBuffer(4 << 20) if buffered else None)
                    theirs = ref_ops.compress(x, dist_of(rf, spec),
                                              RefBuffer(4 << 20, device="cuda") if buffered else None)
                    by_reference = ref_ops.decompress(translate(ours, RefTensor, rf))
                    by_this = our_ops.decompress(translate(theirs, OurTensor, of))
                    key = f"{backend}/{name}/{'arena' if buffered else 'private'}"
                    report["cases"][key] = {
                        "overflow_streams": int(ours.fallback_count.item()),
                        "reference_decodes_ours": bool(torch.equal(by_reference.view(torch.int16),
                                                                   x.view(torch.int16))),
                        "this_decodes_reference": bool(torch.equal(by_this.view(torch.int16),
                                                                   x.view(torch.int16))),
                        "same_memory_size": int(ours.memory_size()) == int(theirs.memory_size()),
                    }
        except Exception as error:
            if backend == "generic":
                raise
            report["a100"] = f"unavailable: {type(error).__name__}: {error}"[:300]
        finally:
            ref_dispatch.backend_for = stock
    report.setdefault("a100", "ran")
    torch.cuda.synchronize()
    with open(args.out, "w") as handle:
        json.dump(report, handle)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("mode", choices=("bits", "bench", "dropin", "interchange"))
    parser.add_argument("--out", required=True)
    parser.add_argument("--sizes", default="1024x1024,4096x4096")
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--iters", type=int, default=20)
    parser.add_argument("--elements", type=int, default=4_000_000)
    parser.add_argument("--autotune", action="store_true")
    args = parser.parse_args()
    if not available():
        raise SystemExit("baseline/_ref is missing: run __graft_entry__.build() where the "
                         "reference checkout exists")
    {"bits": mode_bits, "bench": mode_bench, "dropin": mode_dropin,
     "interchange": mode_interchange}[args.mode](args)


if __name__ == "__main__":
    main()
