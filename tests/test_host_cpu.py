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


def test_caching_allocator_policy(torch_gcu):
    r = torch_gcu._C._allocator_selftest()
    assert r["round_small"] == 1024 and r["round_large"] == 2 << 20
    assert r["same_stream_reuse"] and r["backend_allocs_after_reuse"] == 1
    assert r["cross_stream_no_reuse"]
    assert r["cached_block_back"] and r["deferred_not_reused"] and r["deferred_reused_after_event"]
    assert r["oom_retry_succeeded"] and r["num_alloc_retries"] >= 1
    assert r["oom_raises"] and r["num_ooms"] == 1
    assert r["capture_ignores_general_cache"] and r["capture_reuses_own_block"]
    assert r["eager_does_not_get_pool_block"] and r["eager_gets_general_block"]
    assert r["plain_allocs_in_capture"] == 2 and r["plain_frees_after_release"] == 1
    assert r["plain_frees_after_output_died"] == 2
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
