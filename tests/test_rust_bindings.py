"""The Rust side is shipped as source (no Rust toolchain on the build machine), so what a compiler
would catch at the FFI seam is checked here mechanically:
  * every function of include/wgf.h is declared in rust/wgf-sys/src/lib.rs with the same parameter
    count and the same parameter and return types, and nothing else is declared there;
  * the constants of the header have the same values in wgf-sys;
  * every `sys::wgf_*` call in rust/wgpu-compute passes as many arguments as the header declares;
  * every public item of the original crate's API (src/lib.rs:1-11 there, and the methods its
    modules add to Tensor) has a counterpart in rust/wgpu-compute."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "wgf.h")
SYS = os.path.join(ROOT, "rust", "wgf-sys", "src", "lib.rs")
FACADE = os.path.join(ROOT, "rust", "wgpu-compute", "src")

PRIM = {"int32_t": "i32", "uint32_t": "u32", "int64_t": "i64", "uint64_t": "u64", "float": "f32", "uint16_t": "u16",
        "uint8_t": "u8", "void": "c_void", "char": "c_char"}


def strip_c_comments(text):
    return re.sub(r"/\*.*?\*/", " ", text, flags=re.S)


def rust_type(c_type):
    """`const wgf_tensor_desc*` -> `*const wgf_tensor_desc`; `wgf_tensor* const*` -> `*const *mut wgf_tensor`."""
    m = re.match(r"^(const\s+)?(\w+)\s*((?:\*\s*(?:const\s*)?)*)$", c_type.strip())
    assert m, c_type
    leading_const, base, stars = m.group(1), m.group(2), m.group(3)
    out = PRIM.get(base, base)
    quals = re.findall(r"\*\s*(const)?", stars)
    for i, _ in enumerate(quals):
        pointee_const = leading_const is not None if i == 0 else quals[i - 1] == "const"
        out = ("*const " if pointee_const else "*mut ") + out
    return out


def header_functions():
    body = strip_c_comments(open(HEADER).read())
    fns = {}
    for ret, name, params in re.findall(r"^(const char\*|int32_t)\s+(wgf_\w+)\s*\(([^;]*?)\)\s*;", body, flags=re.M | re.S):
        params = " ".join(params.split())
        types = []
        if params != "void":
            for p in params.split(","):
                p = p.strip()
                arr = re.match(r"^(.*?)(\w+)\s*\[\w+\]$", p)
                if arr:
                    types.append(rust_type(arr.group(1).strip() + "*"))
                else:
                    types.append(rust_type(re.match(r"^(.*?)(\w+)$", p).group(1)))
        fns[name] = (types, "*const c_char" if ret.startswith("const char") else "i32")
    return fns


def sys_functions():
    text = re.sub(r"//[^\n]*", "", open(SYS).read())
    block = text[text.index('extern "C" {'):]
    fns = {}
    for name, params, ret in re.findall(r"pub fn (wgf_\w+)\s*\((.*?)\)\s*->\s*([^;]+);", block, flags=re.S):
        types = [" ".join(p.split(":", 1)[1].split()) for p in params.split(",") if ":" in p]
        fns[name] = (types, " ".join(ret.split()))
    return fns


def test_every_header_function_is_declared_in_wgf_sys_with_the_same_signature():
    h, r = header_functions(), sys_functions()
    assert len(h) >= 80
    assert sorted(h) == sorted(r), f"only in the header: {sorted(set(h) - set(r))}; only in wgf-sys: {sorted(set(r) - set(h))}"
    for name in h:
        assert h[name] == r[name], f"{name}: header {h[name]} vs wgf-sys {r[name]}"


def test_constants_agree():
    body = strip_c_comments(open(HEADER).read())
    values = {}
    for block in re.findall(r"enum\s*\{(.*?)\};", body, flags=re.S):
        nxt = 0
        for item in block.split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                name, v = [t.strip() for t in item.split("=")]
                nxt = int(v, 0)
            else:
                name = item
            values[name] = nxt
            nxt += 1
    for name, v in re.findall(r"#define\s+(WGF_\w+)\s+(\d+)", body):
        values[name] = int(v)
    rust = dict((n, int(v)) for n, v in re.findall(r"pub const (WGF_\w+): \w+ = (\d+);", open(SYS).read()))
    assert len(values) >= 50
    for name, v in values.items():
        assert rust.get(name) == v, f"{name}: header {v}, wgf-sys {rust.get(name)}"


def split_top_level(args):
    parts, depth, cur = [], 0, ""
    for ch in args:
        if ch in "([{<":
            depth += 1
        elif ch in ")]}>":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        parts.append(cur)
    return parts


def test_facade_calls_match_the_header_arity():
    h = header_functions()
    calls = 0
    used = set()
    for fname in sorted(os.listdir(FACADE)):
        text = re.sub(r"//[^\n]*", "", open(os.path.join(FACADE, fname)).read())
        for m in re.finditer(r"(?:sys|wgf_sys)::(wgf_\w+)\s*\(", text):
            name = m.group(1)
            i, depth = m.end(), 1
            while depth:
                depth += {"(": 1, ")": -1}.get(text[i], 0)
                i += 1
            args = split_top_level(text[m.end():i - 1])
            assert name in h, f"{fname}: {name} is not in the header"
            assert len(args) == len(h[name][0]), f"{fname}: {name} called with {len(args)} arguments, declared with {len(h[name][0])}"
            calls += 1
            used.add(name)
    assert calls >= 60
    # the graph-level API and the device are all reachable from the Rust side
    graph_level = {n for n in h if n.startswith(("wgf_tensor_", "wgf_device_create", "wgf_schedule_", "wgf_comm_"))}
    # (arange runs its loop on the host in the element type, like the original: no call)
    unreachable = graph_level - used - {"wgf_tensor_from_host_pinned", "wgf_tensor_from_desc", "wgf_tensor_timing_labels",
                                       "wgf_tensor_graph_size", "wgf_tensor_arange"}
    assert not unreachable, f"not used by the facade: {sorted(unreachable)}"


def test_public_surface_of_the_original_crate_has_counterparts():
    src = "\n".join(open(os.path.join(FACADE, f)).read() for f in sorted(os.listdir(FACADE)))
    for item in ["pub struct Device", "pub struct Tensor<const R: usize, D>", "pub struct TensorSlice<const R: usize, D>",
                 "pub trait DataType", "pub enum DataTypeEnum", "pub trait IntoTensor<const R: usize, D>",
                 "pub struct Layout", "pub struct QueryResults", "pub struct PerformanceQueries", "pub struct ReduceFunction",
                 "pub trait CastTensor<T>", "pub trait Unsqueeze", "pub trait Sum", "pub trait Max", "pub trait Min",
                 "pub trait Product", "pub async fn new()", "pub fn wgpu_device(", "pub async fn as_slice(",
                 "pub async fn all_timing_information(", "pub fn shape(", "pub fn rank(", "pub fn datatype(", "pub fn graphvis(",
                 "pub fn new(device: &Device, data: impl IntoTensor<R, D>)", "pub fn arange(", "pub fn arange_step(",
                 "pub fn cat(", "pub fn narrow(", "pub fn silu(", "pub fn layer_norm(", "pub fn softmax(", "pub fn rope(",
                 "pub fn mat_mul(", "pub fn slice(", "pub fn transpose(", "pub fn broadcast<const R2: usize>(",
                 "pub fn resize(", "pub fn reshape<const R2: usize>(", "pub fn slice_assign(", "pub fn pow(", "pub fn cast<T2>(",
                 "pub fn contiguous(", "pub fn from_parts(", "pub fn is_contiguous(", "pub fn strides(", "pub fn offset(",
                 "pub fn elapsed(", "pub fn get(", "impl<const R: usize, D: DataType> Neg for Tensor<R, D>"]:
        assert item in src, f"missing in rust/wgpu-compute: {item}"
    unary = re.search(r"unary_functions!\((.*?)\);", src, flags=re.S).group(1)
    for fn in ["exp", "exp2", "log", "log2", "sqr", "sqrt", "sin", "cos", "tan", "asin", "acos", "atan", "sinh", "cosh", "tanh",
               "asinh", "acosh", "atanh", "abs"]:
        assert re.search(rf"\b{fn} =>", unary), f"unary function {fn} missing"
    for trait_, method in [("Add", "add"), ("Sub", "sub"), ("Mul", "mul"), ("Div", "div")]:
        assert f"scalar_operator!({trait_}, {method}," in src and f"pair_operator!({trait_}, {method}," in src
    # the original's example, restated
    hello = open(os.path.join(ROOT, "rust", "wgpu-compute", "examples", "hello.rs")).read()
    for line in ["Device::new().await.unwrap()", "device.wgpu_device().poll(wgpu::PollType::Wait).unwrap()",
                 "Tensor::new(&device, &vec![vec![[1.; 20]; 10]; 10])", "tensor.sum(0).sum(0).sum(0)",
                 "new.all_timing_information().await"]:
        assert line in hello
