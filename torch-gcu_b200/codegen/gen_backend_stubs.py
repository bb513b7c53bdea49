"""Code generator of the PrivateUse1 ("gcu") dispatcher registrations.

    python codegen/gen_backend_stubs.py [--yaml gcu_native_functions.yaml] [--out DIR]

It keeps the reference generator's contract (reference: codegen/gen_backend_stubs.py
:run():742-1143, parse_backend_yaml:77-339, wrapper_torch_codegen.py:248-444,
gen_structured.py:122-206): the operator list lives in `gcu_native_functions.yaml`
(`backend`, `cpp_namespace`, `supported` rows with per-op flags), schemas and
C++ signatures come from PyTorch's own packaged `native_functions.yaml` through
torchgen, and the output is

  RegisterGCU.cpp      TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) { m.impl(...) ... }
                       plus one wrapper per row; structured `.out` operators get a
                       subclass of ATen's own `at::meta::structured_<op>` whose
                       set_output_* overrides allocate / resize on the device, so
                       shapes, dtypes and strides are CPU-identical by construction
  gcu_aot_ops_gen.h    declarations of the `torch_gcu::aotops::<op>` functions
                       the wrappers call (hand-written in csrc/host/aten/*.cpp)

What changed against the reference is what the wrappers call: one hop into
`aotops::<op>`, which marshals into the C ABI of the kernel library; there is no
debug/fallback/op-check wrapper chain and no CPU fallback.
"""
import argparse
import os

import yaml
from torchgen.api import cpp
from torchgen.api import meta as meta_api
from torchgen.api.types import DispatcherSignature
from torchgen.gen import get_grouped_native_functions, parse_native_yaml
from torchgen.context import native_function_manager
from torchgen.model import NativeFunctionsGroup

HERE = os.path.dirname(os.path.abspath(__file__))
ROW_FLAGS = {"name", "kernel_name", "device_guard", "device_check", "disable", "gen_aot_ops",
             "support_deterministic_algorithms", "dynamic_output_shape", "fallback_cpu", "op_check",
             "topsaten_name", "gen_native_function", "gen_topsaten_bridge"}


def parse_backend_yaml(path):
    with open(path) as f:
        doc = yaml.safe_load(f)
    assert doc.get("backend") == "GCU", "backend must be GCU"
    ns = doc.get("cpp_namespace", "torch_gcu")
    rows = []
    for row in doc.get("supported", []) + doc.get("optional", []):
        if isinstance(row, str):
            row = {"name": row}
        unknown = set(row) - ROW_FLAGS
        assert not unknown, "unknown flags %s in row %s" % (unknown, row)
        if row.get("disable"):
            continue
        rows.append(row)
    return ns, rows


def load_native_functions():
    import torchgen
    base = os.path.join(os.path.dirname(torchgen.__file__), "packaged", "ATen", "native")
    parsed = parse_native_yaml(os.path.join(base, "native_functions.yaml"), os.path.join(base, "tags.yaml"))
    by_name = {str(f.func.name): f for f in parsed.native_functions}
    groups = {}
    for g in get_grouped_native_functions(parsed.native_functions):
        if isinstance(g, NativeFunctionsGroup):
            for f in g.functions():
                groups[str(f.func.name)] = g
    return by_name, groups


def cpp_name(f):
    return f.func.name.unambiguous_name()


def first_tensor_arg(sig):
    for a in sig.arguments():
        t = a.type
        if "Tensor" in t and "optional" not in t.lower() and "List" not in t:
            return a.name
    for a in sig.arguments():
        if "TensorList" in a.type or "ITensorListRef" in a.type:
            return a.name + ".front()" if "ITensorListRef" not in a.type else "*%s.begin()" % a.name
    return None


def gen_unstructured(f, row, ns):
    sig = DispatcherSignature.from_schema(f.func, symint=False)
    name = cpp_name(f)
    args = sig.arguments()
    decl_args = ", ".join("%s %s" % (a.type, a.name) for a in args)
    call_args = ", ".join(a.name for a in args)
    ret = sig.returns_type().cpp_type()
    guard = ""
    if row.get("device_guard", True):
        t = first_tensor_arg(sig)
        if t:
            guard = "  const c10::OptionalDeviceGuard device_guard(at::device_of(%s));\n" % t
        elif any(a.name == "device" for a in args):
            guard = "  const c10::OptionalDeviceGuard device_guard(device);\n"
    decl = "%s %s(%s);" % (ret, name, decl_args)
    wrapper = ("%s wrapper_GCU_%s(%s) {\n%s  return %s::aotops::%s(%s);\n}\n" %
               (ret, name, decl_args, guard, ns, name, call_args))
    return decl, wrapper


def gen_structured(f, g, row, ns):
    """f is the out variant of a structured group."""
    sig = DispatcherSignature.from_schema(f.func, symint=False)
    name = cpp_name(f)
    meta_name = "at::meta::structured_" + meta_api.name(g)
    args = sig.arguments()
    n_out = len(f.func.arguments.out)
    out_names = [a.name for a in f.func.arguments.out]
    decl_args = ", ".join("%s %s" % (a.type, a.name) for a in args)
    in_args = [a for a in args if a.name not in out_names]
    # meta() takes the functional arguments in schema order (as the structured C++ API spells them)
    def meta_arg(a):
        # the structured API spells optional scalars as a non-owning reference
        if "optional<at::Scalar>" in str(a.type):
            return "(%s.has_value() ? at::OptionalScalarRef(&(%s.value())) : at::OptionalScalarRef())" % (a.name, a.name)
        if "optional<at::Tensor>" in str(a.type) and "List" not in str(a.type):
            return "((%s.has_value() && %s->defined()) ? at::OptionalTensorRef(*%s) : at::OptionalTensorRef())" % (a.name, a.name, a.name)
        return a.name
    meta_call = ", ".join(meta_arg(a) for a in in_args)
    inherits_iter = g.out.structured_inherits is not None
    precomputed = g.out.precomputed is not None
    cls = "structured_%s_gcu" % name
    super_call = ("    %s::set_output_raw_strided(output_idx, sizes, strides, options, names);\n" % meta_name
                  if inherits_iter else "")
    klass = """struct {cls} final : public {meta} {{
  {cls}({ctor_args}) : outputs_{{ {refs} }} {{}}
  void set_output_strided(int64_t output_idx, at::IntArrayRef sizes, at::IntArrayRef strides,
                          at::TensorOptions options, at::DimnameList names) override {{
    const at::Tensor& out = outputs_[output_idx].get();
    {ns}::resize_out(out, sizes, strides, options);
    auto proxy = {ns}::maybe_create_proxy(out, sizes, strides, options);
    if (proxy.has_value()) proxy_outputs_[output_idx] = std::move(proxy).value();
    (void)names;
{super}  }}
  void set_output_raw_strided(int64_t output_idx, at::IntArrayRef sizes, at::IntArrayRef strides,
                              at::TensorOptions options, at::DimnameList names) override {{
    const at::Tensor& out = outputs_[output_idx].get();
    {ns}::resize_out(out, sizes, strides, options);
    (void)names;
{super}  }}
  const at::Tensor& maybe_get_output(int64_t output_idx) override {{
    return proxy_outputs_[output_idx].has_value() ? *proxy_outputs_[output_idx] : outputs_[output_idx].get();
  }}
  std::array<std::reference_wrapper<at::Tensor>, {n}> outputs_;
  std::array<std::optional<at::Tensor>, {n}> proxy_outputs_;
}};
""".format(cls=cls, meta=meta_name, ns=ns, n=n_out, super=super_call,
           ctor_args=", ".join("at::Tensor& out%d" % i for i in range(n_out)),
           refs=", ".join("std::ref(out%d)" % i for i in range(n_out)))
    impl_args = []
    if inherits_iter:
        impl_args.append("at::TensorIteratorBase& iter")
    if precomputed:
        impl_args.append("const %s::meta_return_ty& precompute" % meta_name)
    impl_args += ["%s %s" % (a.type, a.name) for a in in_args]
    impl_args += ["const at::Tensor& %s" % o for o in out_names]
    decl = "void %s(%s);" % (name, ", ".join(impl_args))
    call = []
    if inherits_iter:
        call.append("op")
    if precomputed:
        call.append("precompute")
    call += [a.name for a in in_args]
    call += ["op.maybe_get_output(%d)" % i for i in range(n_out)]
    ret = sig.returns_type().cpp_type()
    if n_out == 1:
        ret_stmt = "  return %s;\n" % out_names[0]
    else:
        ret_stmt = "  return std::forward_as_tuple(%s);\n" % ", ".join(out_names)
    copy_back = "".join(
        "  if (op.proxy_outputs_[%d].has_value()) op.outputs_[%d].get().copy_(*op.proxy_outputs_[%d]);\n" % (i, i, i)
        for i in range(n_out))
    guard = "  const c10::OptionalDeviceGuard device_guard(at::device_of(%s));\n" % out_names[0]
    meta_stmt = ("  auto precompute = op.meta(%s);\n  (void)precompute;\n" if precomputed else "  op.meta(%s);\n") % meta_call
    wrapper = ("%s wrapper_GCU_%s(%s) {\n%s  %s op(%s);\n%s  %s::aotops::%s(%s);\n%s%s}\n" %
               (ret, name, decl_args, guard, cls, ", ".join(out_names), meta_stmt, ns, name, ", ".join(call),
                copy_back, ret_stmt))
    return decl, klass + wrapper


def run(yaml_path, out_dir):
    ns, rows = parse_backend_yaml(yaml_path)
    by_name, groups = load_native_functions()
    decls, bodies, impls, meta_headers = [], [], [], []
    for row in rows:
        name = row["name"]
        assert name in by_name, "%s is not an ATen operator of this PyTorch" % name
        f = by_name[name]
        g = groups.get(name)
        with native_function_manager(f):
            if g is not None and g.structured and f is g.out:
                decl, body = gen_structured(f, g, row, ns)
                inc = "#include <ATen/ops/%s_meta.h>" % g.root_name
                if inc not in meta_headers:
                    meta_headers.append(inc)
            else:
                decl, body = gen_unstructured(f, row, ns)
        decls.append(decl)
        bodies.append(body)
        impls.append('  m.impl("%s", TORCH_FN(wrapper_GCU_%s));' % (name, cpp_name(f)))
    os.makedirs(out_dir, exist_ok=True)
    header = ("// @generated by codegen/gen_backend_stubs.py from gcu_native_functions.yaml -- do not edit.\n"
              "#pragma once\n#include <ATen/ATen.h>\n#include <ATen/TensorIterator.h>\n%s\n\n"
              "namespace %s {\nnamespace aotops {\n\n%s\n\n}  // namespace aotops\n}  // namespace %s\n" %
              ("\n".join(meta_headers), ns, "\n".join(decls), ns))
    source = ("// @generated by codegen/gen_backend_stubs.py from gcu_native_functions.yaml -- do not edit.\n"
              "#include <ATen/ATen.h>\n#include <ATen/TensorIterator.h>\n"
              "#include <c10/core/DeviceGuard.h>\n#include <torch/library.h>\n\n"
              '#include "aten/structured_helpers.h"\n#include "aten/generated/gcu_aot_ops_gen.h"\n\n'
              "namespace {\n\n%s\n}  // namespace\n\nTORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {\n%s\n}\n" %
              ("\n".join(bodies), "\n".join(impls)))
    for fname, text in (("gcu_aot_ops_gen.h", header), ("RegisterGCU.cpp", source)):
        path = os.path.join(out_dir, fname)
        if not os.path.exists(path) or open(path).read() != text:
            with open(path, "w") as fh:
                fh.write(text)
    return [r["name"] for r in rows]


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--yaml", default=os.path.join(HERE, "gcu_native_functions.yaml"))
    ap.add_argument("--out", default=os.path.join(os.path.dirname(HERE), "csrc", "host", "aten", "generated"))
    a = ap.parse_args()
    names = run(a.yaml, a.out)
    print("generated %d registrations into %s" % (len(names), a.out))
