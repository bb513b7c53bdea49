"""Host-side logic that needs no GPU: the package imports and registers the
backend, the code generator emits one registration per yaml row, the caching
allocator's policy (against a fake device backend), argument checks of the c10d
backend, and a world-size-2 gloo run of the tensor-parallel sharding logic."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "torch-gcu_b200")


@pytest.fixture(scope="module")
def torch_gcu():
    import torch_gcu
    return torch_gcu


def test_backend_is_registered(torch_gcu):
    assert torch._C._get_privateuse1_backend_name() == "gcu"
    assert hasattr(torch, "gcu") and hasattr(torch.Tensor, "gcu") and hasattr(torch.Tensor, "is_gcu")
    assert torch.gcu.device_count() >= 0
    assert "sm_100a" in torch_gcu._C._kernel_library_version()
    assert torch.distributed.is_eccl_available()
    assert "eccl" in torch.distributed.Backend.backend_list


def test_no_cpu_fallback_without_device(torch_gcu):
    if torch.gcu.is_available():
        pytest.skip("a device is present")
    with pytest.raises(RuntimeError):
        torch.zeros(2, device="gcu")


def test_autocast_state_accessors(torch_gcu):
    prev = torch.gcu.is_autocast_enabled()
    torch.gcu.set_autocast_enabled(True)
    assert torch.gcu.is_autocast_enabled()
    torch.gcu.set_autocast_dtype(torch.bfloat16)
    assert torch.gcu.get_autocast_dtype() == torch.bfloat16
    torch.gcu.set_autocast_enabled(prev)
    with torch.autocast("gcu", dtype=torch.bfloat16):
        assert torch.is_autocast_enabled("gcu")
    assert isinstance(torch.gcu.amp.autocast(), torch.amp.autocast_mode.autocast)


@pytest.fixture(scope="module")
def selftest():
    """The test-only native module (tests/native): the product's allocator and watchdog sources
    compiled together with fakes of the device and of the communicator."""
    import importlib.util
    import torch  # noqa: F401  (its libraries must be loaded first)
    path = os.path.join(ROOT, "tests", "native", "_gcu_selftest.so")
    assert os.path.exists(path), "tests/native/_gcu_selftest.so is built by __graft_entry__.build()"
    spec = importlib.util.spec_from_file_location("_gcu_selftest", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_product_extension_carries_no_test_harness(torch_gcu):
    assert not hasattr(torch_gcu._C, "_allocator_selftest")


def test_caching_allocator_policy(selftest):
    r = selftest.allocator_selftest()
    assert r["round_small"] == 1024 and r["round_large"] == 2 << 20
    assert r["same_stream_reuse"] and r["backend_allocs_after_reuse"] == 1
    assert r["cross_stream_no_reuse"]
    assert r["cached_block_back"] and r["deferred_not_reused"] and r["deferred_reused_after_event"]
    assert r["oom_retry_succeeded"] and r["num_alloc_retries"] >= 1
    assert r["oom_raises"] and r["num_ooms"] == 1
    assert r["capture_ignores_general_cache"] and r["capture_reuses_own_block"]
    assert r["eager_does_not_get_pool_block"] and r["eager_gets_general_block"]
    assert r["plain_allocs_in_capture"] == 2 and r["plain_frees_after_release"] == 1
    assert r["plain_frees_after_output_died"] == 2   # the last live block of a released pool (pool erased after it)
    assert r["no_event_recorded_during_capture"] and r["event_recorded_after_capture"]
    assert r["parked_block_not_reused_early"] and r["parked_block_reused_after_event"]
    assert r["side_stream_allocates_from_pool"] and r["no_cross_stream_reuse_inside_pool"]
    assert r["same_stream_reuse_inside_pool"]
    assert r["allocated_after_all_freed"] == 0 and r["reserved_after_empty_cache"] == 0
    assert r["backend_outstanding"] == 0 and r["cache_hits"] >= 3


def test_codegen_emits_every_row(tmp_path):
    sys.path.insert(0, os.path.join(PKG, "codegen"))
    import gen_backend_stubs as gen
    names = gen.run(os.path.join(PKG, "codegen", "gcu_native_functions.yaml"), str(tmp_path))
    src = (tmp_path / "RegisterGCU.cpp").read_text()
    hdr = (tmp_path / "gcu_aot_ops_gen.h").read_text()
    assert "TORCH_LIBRARY_IMPL(aten, PrivateUse1, m)" in src
    for n in names:
        assert 'm.impl("%s"' % n in src
    for must in ("add.out", "mul.out", "silu.out", "sum.IntList_out", "_softmax.out", "native_layer_norm",
                 "index_select", "gather.out", "scatter_add.out", "_index_put_impl_", "mm.out", "addmm.out", "bmm.out",
                 "_scaled_dot_product_flash_attention", "_copy_from", "empty.memory_format", "empty_strided"):
        assert must in names
    # structured rows reuse ATen's own meta classes
    assert "public at::meta::structured_add_Tensor" in src
    assert "void add_out(at::TensorIteratorBase& iter" in hdr
    # the committed generated files are what the generator produces today
    committed = open(os.path.join(PKG, "csrc", "host", "aten", "generated", "RegisterGCU.cpp")).read()
    assert committed == src


def test_codegen_rejects_unknown_rows(tmp_path):
    sys.path.insert(0, os.path.join(PKG, "codegen"))
    import gen_backend_stubs as gen
    bad = tmp_path / "bad.yaml"
    bad.write_text("backend: GCU\ncpp_namespace: torch_gcu\nsupported:\n- name: not_an_op.out\n")
    with pytest.raises(AssertionError):
        gen.run(str(bad), str(tmp_path))


def test_process_group_argument_checks(torch_gcu):
    PG = torch_gcu._C._distributed_c10d.ProcessGroupECCL
    with pytest.raises(RuntimeError, match="gcu device"):
        PG._check_tensor(torch.zeros(4))
    store = torch.distributed.HashStore()
    with pytest.raises(RuntimeError, match="invalid rank"):
        PG(store, 3, 2, PG.Options())
    pg = PG(store, 0, 1, PG.Options())
    assert pg.options.is_high_priority_stream
    with pytest.raises(RuntimeError):  # host tensors are rejected before anything is launched
        pg.allreduce([torch.zeros(4)])
    pg.shutdown()


def _wait_until(cond, seconds=5.0):
    import time
    end = time.monotonic() + seconds
    while time.monotonic() < end:
        if cond():
            return True
        time.sleep(0.01)
    return cond()


def test_watchdog_times_out_a_work_that_never_completes(selftest):
    """Failure made on the host: a collective whose completion query never turns true. After its
    100 ms timeout the watchdog sets the work's exception, aborts the communicator exactly once,
    fails what else was outstanding, and refuses later works (reference: checkTimeout /
    watchdogHandler, torch_gcu/csrc/distributed/ProcessGroupECCL.cpp:533-556, :1485-1616)."""
    aborts = []
    wd = selftest.Watchdog(lambda: "", lambda: aborts.append(1), 10)
    try:
        done = selftest.FakeWork(lambda: True, 100, 1)
        stuck = selftest.FakeWork(lambda: False, 100, 2)
        bystander = selftest.FakeWork(lambda: False, 60_000, 3)   # far from its own timeout
        for w in (done, stuck, bystander):
            wd.watch(w)
        assert _wait_until(lambda: done.finished)
        assert not done.failed and done.exception_text == ""
        assert _wait_until(lambda: wd.has_failed and wd.abort_calls == 1 and wd.outstanding() == 0)
        assert "DistBackendError" in stuck.exception_text
        assert "collective (seq 2) did not complete within 100 ms" in stuck.exception_text
        assert not stuck.finished
        assert "seq 3" in bystander.exception_text and "communicator was aborted" in bystander.exception_text
        assert "seq 2" in bystander.exception_text      # carries the cause
        assert "seq 2" in wd.failure()
        late = selftest.FakeWork(lambda: True, 100, 4)
        with pytest.raises(RuntimeError, match="aborted after an earlier failure"):
            wd.watch(late)
        assert late.failed and wd.outstanding() == 0
        import time
        time.sleep(0.1)
        assert aborts == [1] and wd.abort_calls == 1     # the abort hook ran once, not once per sweep
    finally:
        wd.stop()


def test_watchdog_turns_an_async_communicator_error_into_the_works_exception(selftest):
    """The communicator's asynchronous-error poll (ncclCommGetAsyncError in the product) answers
    with an error while two works are out: both fail with that text, one abort (reference:
    checkForECCLErrors, ProcessGroupECCL.cpp:1682-1700)."""
    state = {"err": ""}
    aborts = []
    wd = selftest.Watchdog(lambda: state["err"], lambda: aborts.append(1), 10)
    try:
        a = selftest.FakeWork(lambda: False, 60_000, 7)
        b = selftest.FakeWork(lambda: False, 60_000, 8)
        wd.watch(a)
        wd.watch(b)
        import time
        time.sleep(0.1)
        assert not wd.has_failed and wd.outstanding() == 2 and not a.failed
        state["err"] = "unhandled system error (fake: peer closed the connection)"
        assert _wait_until(lambda: wd.has_failed and wd.abort_calls == 1)
        for w, seq in ((a, 7), (b, 8)):
            assert "asynchronous error" in w.exception_text and "peer closed the connection" in w.exception_text
            assert "seq %d" % seq in w.exception_text
        assert aborts == [1]
        with pytest.raises(RuntimeError, match="peer closed the connection"):
            wd.watch(selftest.FakeWork(lambda: True, 100, 9))
    finally:
        wd.stop()


def test_tensor_parallel_sharding_gloo_world2():
    """The TP harness's host logic (weight sharding + allreduce of row-parallel
    partial sums) on two CPU ranks over gloo reproduces the unsharded layer."""
    script = os.path.join(ROOT, "tests", "tp_gloo_worker.py")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29617")
    procs = [subprocess.Popen([sys.executable, script, str(r), "2"], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
    assert "TP_OK" in outs[0]
