"""The host layer on the B200 device, and raw SSA kernels through
ugb_compile / ugb_run.  The lazy-graph cases are the reference's fixtures
(tests/lazy_cases.py); graph results are compared with the same graphs run on
the CPU oracle device (fp32 reductions <= 1e-5 relative, copies bit-exact)."""
import numpy as np
import pytest

import lazy_cases as cases
import oracle
from conftest import rel_err
from oracle import llama_ref as R
from ug_b200 import DType, UgError, synth
from ug_b200.lazy import LB, BinaryOp as B, HostDevice, ReduceOp as Rd, Schedule, UnaryOp as U, ssa
from ug_b200.llama import Config

pytestmark = pytest.mark.gpu
I = ssa.instr


@pytest.fixture(scope="module")
def hdev(dev):
    return HostDevice(dev)


@pytest.fixture(scope="module")
def cpu():
    return oracle.cpu_host_device()


@pytest.fixture(params=["b200_policy", "reference_policy"])
def policy(request, hdev):
    hdev.set_launch_policy(request.param == "reference_policy")
    yield request.param
    hdev.set_launch_policy(False)


@pytest.mark.parametrize("case", ["add", "mm", "cat", "schedule_one_kernel", "lb_copy", "schedule_broadcast",
                                  "lb_layout", "lb_set", "errors", "cache_hits"])
def test_reference_fixtures(hdev, policy, case):
    getattr(cases, case)(hdev)
    hdev.synchronize()


def test_custom_ops(hdev, dev):
    ones = dev.slice_from_values(np.ones(6, np.float32))

    def add_one(s):
        dev.add(hdev.ops._s(s[0]), ones, hdev.ops._s(s[1]), 6)

    def add_one_ip(s):
        dev.add(hdev.ops._s(s[0]), ones, hdev.ops._s(s[0]), 6)
    cases.custom_ops(hdev, add_one, add_one_ip)


def test_layout_chain(hdev, policy):
    cases.layout_chain(hdev, synth.normal(1, (2, 5, 16)))


@pytest.mark.parametrize("rows,cols", [(2, 4), (6, 300), (64, 256), (33, 1024), (5, 4096), (3, 777)])
def test_graph_softmax_and_rms_silu_match_the_cpu_backend(hdev, cpu, policy, rows, cols):
    if policy == "reference_policy" and rows * cols * cols > 2 ** 24:
        pytest.skip("the reference launch shape re-runs the reduction per element: too slow to be useful")
    x = synth.normal(2 + cols, (rows, cols), 2.0)
    assert rel_err(cases.graph_softmax(hdev, x), cases.graph_softmax(cpu, x)) < 1e-5
    g = synth.normal(3 + cols, (rows, cols))
    w = synth.uniform(4 + cols, (cols,), 0.5, 1.5)
    got, items = cases.graph_rms_silu(hdev, x, w, g)
    want, _ = cases.graph_rms_silu(cpu, x, w, g)
    assert items == ["Kernel"]
    assert rel_err(got, want, 1e-20) < 1e-5


def test_b200_policy_hoists_row_reductions(hdev):
    """This backend's lowering of a row softmax: one block per row, 256 threads striding the row, the max /
    sum evaluated once per row by a block reduction (the reference's shape re-runs them per element)."""
    hdev.set_launch_policy(False)
    x = LB.copy(synth.normal(5, (64, 1000)), (64, 1000), hdev)
    from ug_b200 import llama_graph as G
    s = Schedule.create_one(G.softmax(x))
    # exp(x - max) has two users, both inside this kernel: this backend evaluates it in place instead of cutting
    # it out (the reference's rule, schedule.rs:429-435, gives two kernels); the max therefore appears in the
    # sum and in the final map, each time hoisted to one block reduction per row
    assert s.items() == ["Kernel"]
    ours, ref = s.ssa_text(0, policy=1), s.ssa_text(0, policy=0)
    assert "launch grid=64 block=256" in ours and ours.count("reduce_local.max") >= 1 and ours.count("reduce_local.sum") == 1
    assert "reduce_local" not in ref
    pure_map = Schedule.create_one(x.unary(U.Exp).binary(B.Mul, x))
    assert "launch grid=250 block=256" in pure_map.ssa_text(0, policy=1)     # 64000 elements, one thread each
    assert "launch grid=1 block=1" in pure_map.ssa_text(0, policy=0)         # the reference: a single thread


def test_llama_graph_on_b200_matches_the_cpu_oracle(hdev):
    from ug_b200 import llama_graph as G
    cfg = Config(hidden_size=64, intermediate_size=96, max_position_embeddings=32, num_attention_heads=4,
                 num_key_value_heads=2, num_hidden_layers=2, vocab_size=50)
    w = synth.llama_weights_f32(synth.llama_weights(cfg))
    ref = R.Model(R.Config(**cfg.__dict__), w, custom_softmax_op=False)
    toks = synth.tokens(6, (1, 7), cfg.vocab_size)
    for custom in (False, True):
        model = G.Model(cfg, w, hdev, custom_softmax_op=custom)
        cache, rcache = model.new_cache(), ref.new_cache()
        for lo, hi in ((0, 5), (5, 6), (6, 7)):
            t = LB.copy(toks[:, lo:hi], (1, hi - lo), hdev)
            pos = LB.copy(np.array([[lo]], np.int32), (1, 1), hdev)
            got = model.fwd(t, pos, cache).data_vec().reshape(1, hi - lo, cfg.vocab_size)
            want = ref.fwd(toks[:, lo:hi], lo, rcache)
            assert np.max(np.abs(got - want)) < 1e-4 * np.abs(want).max()    # f32 everywhere, GEMM order differs


# ------------------------------------------------------- raw SSA kernels ----
def test_ssa_simple_add_reference_vector(dev):
    # ug-core/src/samples.rs:10-28 run as ug-core/tests/cpu_tests.rs:3-16 does: [3,1,4,1,5,9] + [1..6]
    i32 = DType.I32
    k = [I("DefineGlobal", i32, index=0), I("DefineGlobal", i32, index=1), I("DefineGlobal", i32, index=2),
         I("Range", a0=ssa.i32(0), a1=ssa.i32(6), index=1, v0=8),
         I("Load", i32, v0=1, a0=3), I("Load", i32, v0=2, a0=3),
         I("Binary", i32, op=B.Add, a0=4, a1=5), I("Store", i32, v0=0, a0=3, a1=6), I("EndRange", v0=3)]
    f = dev.compile(k, name="foo")
    v1 = dev.slice_from_values(np.zeros(6, np.int32))
    v2 = dev.slice_from_values(np.array([3, 1, 4, 1, 5, 9], np.int32))
    v3 = dev.slice_from_values(np.array([1, 2, 3, 4, 5, 6], np.int32))
    dev.run(f, [v1, v2, v3])
    dev.synchronize()
    assert np.array_equal(v1.to_vec(), [4, 3, 7, 5, 10, 15])
    assert '__global__ void ug_foo_' in f.source


def test_ssa_dotprod_reference_vector(dev):
    # ug-core/src/samples.rs:30-52 with the operands of ug-core/tests/basic_tests.rs:15-26 -> 12.0
    f32 = DType.F32
    k = [I("DefineGlobal", f32, index=0), I("DefineGlobal", f32, index=1), I("DefineGlobal", f32, index=2),
         I("Const", cst=ssa.i32(0)), I("Const", cst=ssa.i32(2)), I("DefineAcc", cst=ssa.f32(0.0)),
         I("Range", a0=3, a1=4, index=1, v0=12), I("Load", f32, v0=1, a0=6), I("Load", f32, v0=2, a0=6),
         I("Binary", f32, op=B.Mul, a0=7, a1=8), I("Binary", f32, op=B.Add, a0=9, a1=5), I("Assign", v0=5, a0=10),
         I("EndRange", v0=6), I("Store", f32, v0=0, a0=3, a1=5)]
    f = dev.compile(k)
    a = dev.slice_from_values(np.zeros(1, np.float32))
    b = dev.slice_from_values(np.array([3., 4.5], np.float32))
    c = dev.slice_from_values(np.array([1., 2.], np.float32))
    dev.run(f, [a, b, c])
    dev.synchronize()
    assert a.to_vec()[0] == 12.0


def softmax_reduce_kernel(dim2):
    # ug-core/src/samples.rs:164-187: one block per row, one thread per column, two ReduceLocal
    f32, i32 = DType.F32, DType.I32
    return [I("DefineGlobal", f32, index=0), I("DefineGlobal", f32, index=1),
            I("Special", i32, op=1), I("Special", i32, op=0),
            I("Binary", i32, op=B.Mul, a0=2, a1=ssa.i32(dim2)), I("Binary", i32, op=B.Add, a0=4, a1=3),
            I("Load", f32, v0=0, a0=5), I("ReduceLocal", f32, op=Rd.Max, a0=6),
            I("Binary", f32, op=B.Sub, a0=6, a1=7), I("Unary", f32, op=U.Exp, a0=8),
            I("ReduceLocal", f32, op=Rd.Sum, a0=9), I("Binary", f32, op=B.Div, a0=9, a1=10),
            I("Store", f32, v0=1, a0=5, a1=11)]


def test_ssa_softmax_reduce_reference_vector(dev):
    # ug-core/tests/basic_tests.rs:91-116
    x = np.array([0., 1., 2., 3., 2., 1., 2., 1.], np.float32)
    gold = np.array([0.032058604, 0.08714432, 0.23688284, 0.6439143, 0.3655293, 0.13447072, 0.3655293, 0.13447072], np.float32)
    f = dev.compile(softmax_reduce_kernel(4), grid_dim=2, block_dim=4)
    src, dst = dev.slice_from_values(x), dev.allocate_uninit(DType.F32, 8)
    dev.run(f, [src, dst])
    dev.synchronize()
    assert rel_err(dst.to_vec(), gold) < 3e-7


@pytest.mark.parametrize("rows,cols", [(7, 32), (5, 100), (3, 1000), (2, 1024)])
def test_ssa_softmax_reduce_any_block_size(dev, rows, cols):
    x = synth.normal(20 + cols, (rows, cols), 2.0)
    f = dev.compile(softmax_reduce_kernel(cols), grid_dim=rows, block_dim=cols)
    src, dst = dev.slice_from_values(x), dev.allocate_uninit(DType.F32, x.size)
    dev.run(f, [src, dst])
    dev.synchronize()
    assert rel_err(dst.to_vec().reshape(x.shape), oracle.custom_softmax(x)) < 1e-5


def test_ssa_shared_memory_and_barrier(dev):
    # DefineLocal + Barrier: reverse each block of 64 values through shared memory
    f32, i32 = DType.F32, DType.I32
    k = [I("DefineGlobal", f32, index=0), I("DefineGlobal", f32, index=1), I("DefineLocal", f32, index=64),
         I("Special", i32, op=1), I("Special", i32, op=0),
         I("Binary", i32, op=B.Mul, a0=3, a1=ssa.i32(64)), I("Binary", i32, op=B.Add, a0=5, a1=4),
         I("Load", f32, v0=0, a0=6), I("Store", f32, v0=2, a0=4, a1=7), I("Barrier"),
         I("Binary", i32, op=B.Sub, a0=ssa.i32(63), a1=4), I("Load", f32, v0=2, a0=10), I("Store", f32, v0=1, a0=6, a1=11)]
    f = dev.compile(k, grid_dim=3, block_dim=64)
    x = synth.normal(30, (3, 64))
    src, dst = dev.slice_from_values(x), dev.allocate_uninit(DType.F32, x.size)
    dev.run(f, [src, dst])
    dev.synchronize()
    assert np.array_equal(dst.to_vec().reshape(3, 64), x[:, ::-1])


def test_ssa_out_of_range_access_is_reported_not_faulted(dev):
    i32 = DType.I32
    k = [I("DefineGlobal", i32, index=0), I("Const", cst=ssa.i32(7)), I("Store", i32, v0=0, a0=ssa.i32(1000), a1=1),
         I("Store", i32, v0=0, a0=ssa.i32(2), a1=1)]
    f = dev.compile(k)
    s = dev.slice_from_values(np.zeros(4, np.int32))
    dev.run(f, [s])
    with pytest.raises(UgError) as e:
        dev.synchronize()
    assert e.value.code == 3
    assert np.array_equal(s.to_vec(), [0, 0, 7, 0])       # the in-range store happened, the other was skipped
    dev.synchronize()


def test_ssa_errors(dev):
    i32 = DType.I32
    with pytest.raises(UgError) as e:       # arguments out of order (lang.rs:742-745)
        dev.compile([I("DefineGlobal", i32, index=1)])
    assert e.value.code == 8
    with pytest.raises(UgError) as e:
        dev.compile([I("DefineGlobal", i32, index=0), I("Range", a0=ssa.i32(0), a1=ssa.i32(2), index=1, v0=2)])
    assert e.value.code == 8 and "unmatched" in e.value.msg
    f = dev.compile([I("DefineGlobal", i32, index=0)])
    fl = dev.allocate_uninit(DType.F32, 4)
    with pytest.raises(UgError) as e:       # dtype of a kernel argument
        dev.run(f, [fl])
    assert e.value.code == 2
    with pytest.raises(UgError) as e:       # arity
        dev.run(f, [])
    assert e.value.code == 1
    z = dev.compile([I("DefineGlobal", i32, index=0)], grid_dim=0, block_dim=32)
    n0 = dev.launch_count
    dev.run(z, [dev.allocate_uninit(DType.I32, 4)])        # zero launch dimension: a no-op (runtime.rs:269-277)
    assert dev.launch_count == n0


def test_ssa_exp_samples(dev):
    # ug-core/src/samples.rs:52-71 (one element per thread) and :73-99 (a block walks a row in steps of block_size)
    f32, i32 = DType.F32, DType.I32
    bs = 32
    k = [I("DefineGlobal", f32, index=0), I("DefineGlobal", f32, index=1), I("Special", i32, op=1), I("Special", i32, op=0),
         I("Binary", i32, op=B.Mul, a0=2, a1=ssa.i32(bs)), I("Binary", i32, op=B.Add, a0=4, a1=3),
         I("Load", f32, v0=0, a0=5), I("Unary", f32, op=U.Exp, a0=6), I("Store", f32, v0=1, a0=5, a1=7)]
    x = synth.normal(31, (4, bs))
    src, dst = dev.slice_from_values(x), dev.allocate_uninit(DType.F32, x.size)
    dev.run(dev.compile(k, grid_dim=4, block_dim=bs), [src, dst])
    dev.synchronize()
    assert rel_err(dst.to_vec().reshape(x.shape), np.exp(x.astype(np.float64))) < 1e-6
    dim2 = 96
    k = [I("DefineGlobal", f32, index=0), I("DefineGlobal", f32, index=1), I("Special", i32, op=1), I("Special", i32, op=0),
         I("Binary", i32, op=B.Mul, a0=2, a1=ssa.i32(dim2)), I("Binary", i32, op=B.Add, a0=4, a1=3)]
    for i in range(0, dim2, bs):
        n = len(k)
        k += [I("Binary", i32, op=B.Add, a0=5, a1=ssa.i32(i)), I("Load", f32, v0=0, a0=n),
              I("Unary", f32, op=U.Exp, a0=n + 1), I("Store", f32, v0=1, a0=n, a1=n + 2)]
    x = synth.normal(32, (5, dim2))
    src, dst = dev.slice_from_values(x), dev.allocate_uninit(DType.F32, x.size)
    dev.run(dev.compile(k, grid_dim=5, block_dim=bs), [src, dst])
    dev.synchronize()
    assert rel_err(dst.to_vec().reshape(x.shape), np.exp(x.astype(np.float64))) < 1e-6


def test_ssa_if_mod_min_and_i64(dev):
    # If / EndIf, Mod, Min, Neg and 64-bit integers: dst[i] = i % 3 == 0 ? min(a[i], -a[i]) : a[i]  (i64)
    i32, i64 = DType.I32, DType.I64
    k = [I("DefineGlobal", i64, index=0), I("DefineGlobal", i64, index=1), I("Special", i32, op=0),
         I("Load", i64, v0=0, a0=2), I("Store", i64, v0=1, a0=2, a1=3),
         I("Binary", i32, op=B.Mod, a0=2, a1=ssa.i32(3)),
         I("Binary", i32, op=B.Sub, a0=ssa.i32(1), a1=5),        # 1 - (i % 3): positive only where i % 3 == 0
         I("Binary", i32, op=B.Max, a0=6, a1=ssa.i32(0)),        # condition: non-zero = taken
         I("If", a0=7, v0=12),
         I("Unary", i64, op=U.Neg, a0=3), I("Binary", i64, op=B.Min, a0=3, a1=9), I("Store", i64, v0=1, a0=2, a1=10),
         I("EndIf")]
    a = np.array([5, -7, 2**40, 9, -2**41, 1, 0, 12], np.int64)
    src, dst = dev.slice_from_values(a), dev.allocate_uninit(DType.I64, a.size)
    dev.run(dev.compile(k, grid_dim=1, block_dim=a.size), [src, dst])
    dev.synchronize()
    want = np.where(np.arange(a.size) % 3 == 0, np.minimum(a, -a), a)
    assert np.array_equal(dst.to_vec(), want)


def test_ssa_half_precision_and_unary_ops(dev):
    # Sqrt / Sin / Cos / Id in f32, and 16-bit buffers copied element by element in their own dtype
    f32, bf16, f16, i32 = DType.F32, DType.BF16, DType.F16, DType.I32
    k = [I("DefineGlobal", bf16, index=0), I("DefineGlobal", f16, index=1), I("DefineGlobal", f32, index=2),
         I("DefineGlobal", bf16, index=3), I("DefineGlobal", f16, index=4),
         I("Special", i32, op=0), I("Load", f32, v0=2, a0=5),
         I("Unary", f32, op=U.Sqrt, a0=6), I("Unary", f32, op=U.Sin, a0=6), I("Unary", f32, op=U.Cos, a0=6),
         I("Binary", f32, op=B.Mul, a0=7, a1=8), I("Binary", f32, op=B.Add, a0=10, a1=9), I("Unary", f32, op=U.Id, a0=11),
         I("Store", f32, v0=2, a0=5, a1=12),
         I("Load", bf16, v0=3, a0=5), I("Store", bf16, v0=0, a0=5, a1=14),
         I("Load", f16, v0=4, a0=5), I("Store", f16, v0=1, a0=5, a1=16)]
    x = np.abs(synth.normal(33, (64,))) + 0.1
    src_bf = synth.to_bf16_bits(synth.normal(34, (64,)))
    src_h = synth.normal(35, (64,)).astype(np.float16)
    o_bf = dev.allocate_uninit(DType.BF16, 64)
    o_h = dev.allocate_uninit(DType.F16, 64)
    xs = dev.slice_from_values(x)
    dev.run(dev.compile(k, grid_dim=1, block_dim=64),
            [o_bf, o_h, xs, dev.slice_from_values(src_bf, bf16=True), dev.slice_from_values(src_h)])
    dev.synchronize()
    x64 = x.astype(np.float64)
    assert rel_err(xs.to_vec(), np.sqrt(x64) * np.sin(x64) + np.cos(x64)) < 1e-5
    assert np.array_equal(o_bf.to_vec(), src_bf)
    assert np.array_equal(o_h.to_vec().view(np.float16), src_h)


def test_compile_cu_and_ptx_launch3(dev):
    """Device.compile_cu / compile_ptx and Func.launch3 of the reference's Python module: a caller-written
    kernel over three f32 slices."""
    n = 1000
    cu = r"""
extern "C" __global__ void axpy(const float* a, const float* b, float* c) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < 1000) c[i] = 2.0f * a[i] + b[i];
}
"""
    f = dev.compile_cu(cu, "axpy", grid_dim=(n + 127) // 128, block_dim=128)
    a, b = synth.normal(61, (n,)), synth.normal(62, (n,))
    sa, sb, sc = dev.slice_from_values(a), dev.slice_from_values(b), dev.zeros(n)
    f.launch3(sa, sb, sc)
    dev.synchronize()
    assert np.array_equal(sc.to_vec(), np.float32(2.0) * a + b)
    with pytest.raises(UgError):
        f.launch3(sa, dev.zeros(n - 1), sc)                   # length mismatch
    with pytest.raises(UgError) as e:
        dev.compile_cu("this is not CUDA", "axpy")
    assert e.value.code == 8
    with pytest.raises(UgError) as e:
        dev.compile_cu(cu, "no_such_entry")
    assert e.value.code == 8
    ptx = r"""
.version 8.7
.target sm_100a
.address_size 64
.visible .entry fill7(.param .u64 p0) {
    .reg .b32 %r<4>; .reg .b64 %rd<4>; .reg .f32 %f<2>;
    ld.param.u64 %rd1, [p0];
    cvta.to.global.u64 %rd2, %rd1;
    mov.u32 %r1, %tid.x;
    mul.wide.u32 %rd3, %r1, 4;
    add.s64 %rd2, %rd2, %rd3;
    mov.f32 %f1, 0f40E00000;
    st.global.f32 [%rd2], %f1;
    ret;
}
"""
    g = dev.compile_ptx(ptx, "fill7", grid_dim=1, block_dim=64)
    out = dev.zeros(64)
    dev.run(g, [out])
    dev.synchronize()
    assert np.array_equal(out.to_vec(), np.full(64, 7.0, np.float32))
