"""Parity figures at the FULL sizes of the five workload configurations, as a table.

    python tests/parity_report.py [--configs c1,c2,c3,c4,c5] [--out report.md]

For each op: the GPU result through the C ABI against the CPU oracle (oracle/fdl_oracle.c)
on the same seeded host arrays, and - where the reference has a CUDA kernel for the op and
oracle/_ref/libref.so is present - against that kernel's output on the same device buffers.
Reported per op, in the form its tolerance is stated in:
  exact ops            number of elements whose bits differ (must be 0)
  transcendental       against the reference's CUDA kernel: largest distance in units in the last
                       place (allowed 2; the same CUDA math functions are called, so it is 0);
                       against the glibc twin: largest absolute error (allowed 1e-5, the bound of the
                       reference's own activation test) and, for information only, the ulp distance -
                       CUDA's expf/tanhf are documented to 2 ulp of the true value and glibc's to 1,
                       and 1/(1+e) adds two more roundings, so two correct results can sit 4 ulp
                       apart; gelu's ulp figure is taken on the scale 0.5*|x|, because 1 + tanh(u)
                       cancels for u << 0 and the formula itself promises no more
  sums / means         largest |got - f64| / max(|f64|, ||addends||_2)          (allowed 1e-5)
  softmax / layernorm  largest |got - f64| / max(1, |f64|)                      (allowed 1e-5)
Seeds: one per tensor, 42, 43, 44, ... in order of appearance within a configuration.
The script exits non-zero if any figure is outside its allowance.
"""
import argparse
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402

from fast_dl_b200 import build, capi as fdl  # noqa: E402
from oracle import oracle as orc  # noqa: E402
from oracle import ref  # noqa: E402

ROWS = []
FAILED = []


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


INFO = float("inf")      # a figure that is reported but has no allowance


def record(config, op, against, form, figure, allowed):
    ok = figure <= allowed
    ROWS.append((config, op, against, form, figure, allowed, ok))
    if not ok:
        FAILED.append((config, op, against, figure, allowed))


def differing(got, want):
    got, want = np.ascontiguousarray(got), np.ascontiguousarray(want)
    d = got.view(np.uint32 if got.dtype == np.float32 else np.uint64) != \
        want.view(np.uint32 if want.dtype == np.float32 else np.uint64)
    if got.dtype == np.float32:
        d &= ~(np.isnan(got) & np.isnan(want))
    return int(d.sum())


def exact(config, op, got, want, against="oracle"):
    record(config, op, against, "differing elements", differing(got, want), 0)


def ulps(config, op, got, want, allowed, against="oracle"):
    record(config, op, against, "max ulp", int(orc.ulp_distance(got, want).max()), allowed)


def transcendental_vs_twin(config, name, x, got, want):
    """Absolute error against the glibc twin (checked) and the ulp distance (reported)."""
    g64, w64 = got.astype(np.float64), want.astype(np.float64)
    record(config, name, "oracle (glibc)", "max abs err", float(np.abs(g64 - w64).max()), 1e-5)
    if name.startswith("gelu"):
        scale = np.spacing(np.maximum(np.abs(want), np.abs(0.5 * x)).astype(np.float32)).astype(np.float64)
        record(config, name, "oracle (glibc)", "max err in ulp of max(|ref|, 0.5|x|)",
               float((np.abs(g64 - w64) / scale).max()), INFO)
    else:
        record(config, name, "oracle (glibc)", "max ulp (informational)", int(orc.ulp_distance(got, want).max()), INFO)


def sums(config, op, got, want64, norm, against="oracle (f64)"):
    got, want64, norm = (np.asarray(v, dtype=np.float64) for v in (got, want64, norm))
    record(config, op, against, "max rel err (norm floor)",
           float((np.abs(got - want64) / np.maximum(np.abs(want64), norm)).max()), 1e-5)


def scaled(config, op, got, want64, against="oracle (f64)"):
    got, want64 = np.asarray(got, dtype=np.float64), np.asarray(want64, dtype=np.float64)
    record(config, op, against, "max err / max(1,|ref|)",
           float((np.abs(got - want64) / np.maximum(1.0, np.abs(want64))).max()), 1e-5)


def ref_out_like(t):
    return torch.empty_like(t)


def c1(have_ref):
    n = 1 << 20
    a, b, c = (np.random.default_rng(42 + i).uniform(-1, 1, n).astype(np.float32) for i in range(3))
    ad, bd, cd = dev(a), dev(b), dev(c)
    fused = host(fdl.mul_add_relu(ad, bd, cd))
    exact("c1", "relu(a*b+c), fused entry", fused, orc.mul_add_relu(a, b, c))
    chain = host(fdl.unary(fdl.binary(fdl.binary(ad, bd, fdl.MUL), cd, fdl.ADD), fdl.RELU))
    exact("c1", "relu(a*b+c), three ops", chain, orc.mul_add_relu(a, b, c))
    for name, k in (("add", 0), ("sub", 1), ("mul", 2), ("div", 3)):
        got = fdl.binary(ad, bd, k)
        exact("c1", name, host(got), orc.binary(a, b, k))
        if have_ref:
            r = ref_out_like(ad)
            ref.gpu_elementwise(ad.data_ptr(), bd.data_ptr(), r.data_ptr(), n, k)
            ref.gpu_sync()
            exact("c1", name, host(got), host(r), "reference kernel")
    x = (a * 6).astype(np.float32)
    xd = dev(x)
    for name, k, allowed in (("relu", 0, 0), ("leaky_relu", 1, 0), ("gelu", 2, 2), ("sigmoid", 3, 2), ("tanh", 4, 3)):
        got = fdl.unary(xd, k, 0.01)
        if allowed == 0:
            exact("c1", name, host(got), orc.unary(x, k, 0.01))
        else:
            transcendental_vs_twin("c1", name, x, host(got), orc.unary(x, k, 0.01))
        if have_ref:
            r = ref_out_like(xd)
            ref.gpu_activation(xd.data_ptr(), r.data_ptr(), n, k, 0.01)
            ref.gpu_sync()
            if allowed == 0:
                exact("c1", name, host(got), host(r), "reference kernel")
            else:
                ulps("c1", name, host(got), host(r), 2, "reference kernel")


def c2(have_ref):
    a = np.random.default_rng(42).normal(0, 1, (4096, 4096)).astype(np.float32)
    b = np.random.default_rng(43).normal(0, 1, (1, 4096)).astype(np.float32)
    s = np.random.default_rng(44).uniform(0.5, 2, (4096, 1)).astype(np.float32)
    ad, bd, sd = dev(a), dev(b), dev(s)
    ab = fdl.broadcast_binary(ad, bd, fdl.ADD)
    exact("c2", "A + b[1,4096]", host(ab), a + b)
    exact("c2", "A + b[1,4096]", host(ab), orc.broadcast_binary(a, b, fdl.ADD), "oracle (strided walk)")
    exact("c2", "(A + b) * s[4096,1]", host(fdl.broadcast_binary(ab, sd, fdl.MUL)), (a + b) * s)
    exact("c2", "A * s[4096,1]", host(fdl.broadcast_binary(ad, sd, fdl.MUL)), a * s)
    inplace = ad.clone()
    fdl.add_row_bias_(inplace, bd.reshape(-1))
    exact("c2", "add_row_bias (in place)", host(inplace), a + b)
    if have_ref:
        r = ad.clone()
        ref.gpu_add_row_bias(r.data_ptr(), bd.data_ptr(), 4096, 4096)
        ref.gpu_sync()
        exact("c2", "add_row_bias (in place)", host(inplace), host(r), "reference kernel")


def c3(have_ref):
    x = np.random.default_rng(42).normal(0, 1, (8192, 8192)).astype(np.float32)
    xd = dev(x)
    x64 = x.astype(np.float64)
    sq = x64 * x64
    sums("c3", "sum axis 1", host(fdl.reduce_rows(xd, fdl.REDUCE_SUM)), x64.sum(axis=1), np.sqrt(sq.sum(axis=1)))
    exact("c3", "max axis 1", host(fdl.reduce_rows(xd, fdl.REDUCE_MAX)), x.max(axis=1))
    got = host(fdl.argmax_rows(xd))
    record("c3", "argmax axis 1 (int64)", "oracle", "differing elements", int((got != orc.argmax_rows(x)).sum()), 0)
    ties = x.copy()
    ties[:, 100] = 9.0
    ties[:, 4099] = 9.0
    ties[:, 8191] = 9.0
    got = host(fdl.argmax_rows(dev(ties)))
    record("c3", "argmax axis 1, three-way ties", "lowest index", "differing elements", int((got != 100).sum()), 0)
    sums("c3", "mean axis 0", host(fdl.reduce_cols(xd, fdl.REDUCE_MEAN)), x64.mean(axis=0),
         np.sqrt(sq.sum(axis=0)) / 8192)
    sums("c3", "sum axis 0", host(fdl.reduce_cols(xd, fdl.REDUCE_SUM)), x64.sum(axis=0), np.sqrt(sq.sum(axis=0)))
    exact("c3", "max axis 0", host(fdl.reduce_cols(xd, fdl.REDUCE_MAX)), x.max(axis=0))
    s32, s64 = fdl.full_sum(xd.reshape(-1), want_f64=True)
    sums("c3", "full sum (fp32 result)", host(s32)[0], x64.sum(), np.sqrt(sq.sum()))
    sums("c3", "full sum (f64 result)", host(s64)[0], x64.sum(), np.sqrt(sq.sum()))
    n = 1 << 24
    flat = xd.reshape(-1)[:n].contiguous()
    for name, tree in (("interleave", fdl.TREE_INTERLEAVE), ("address", fdl.TREE_ADDRESS)):
        got = fdl.block_reduce_1024(flat, tree)
        exact("c3", f"1024-block partial sums, {name} tree, n=2^24", host(got),
              orc.block_reduce_1024(x.reshape(-1)[:n], tree))
        if have_ref:
            r = torch.empty(n // 1024, dtype=torch.float32, device="cuda")
            ref.gpu_reduction(flat.data_ptr(), r.data_ptr(), n, tree)
            ref.gpu_sync()
            exact("c3", f"1024-block partial sums, {name} tree, n=2^24", host(got), host(r), "reference kernel")


def c4(have_ref):
    rows, cols = 65536, 1024
    x = np.random.default_rng(42).normal(0, 3, (rows, cols)).astype(np.float32)
    g = np.random.default_rng(43).uniform(0.9, 1.1, cols).astype(np.float32)
    b = np.random.default_rng(44).uniform(-0.1, 0.1, cols).astype(np.float32)
    xd, gd, bd = dev(x), dev(g), dev(b)
    sm = fdl.softmax_rows(xd)
    scaled("c4", "row softmax", host(sm), orc.softmax_rows_f64(x))
    record("c4", "row softmax: |row sum - 1|", "property", "max abs", float((sm.double().sum(dim=1) - 1).abs().max()), 1e-5)
    ln = fdl.layernorm_rows(xd)
    scaled("c4", "layernorm", host(ln), orc.layernorm_rows_f64(x))
    lna = fdl.layernorm_rows(xd, gd, bd)
    scaled("c4", "layernorm + gamma, beta", host(lna), orc.layernorm_rows_f64(x, g, b))
    if have_ref:
        threads = ref.hardware_threads()
        scaled("c4", "row softmax", host(sm), ref.cpu_softmax(x, threads=threads), "reference CPU function")
        scaled("c4", "layernorm", host(ln), ref.cpu_layernorm(x, threads=threads), "reference CPU function")
        r = torch.empty_like(xd)
        ref.gpu_softmax(xd.data_ptr(), r.data_ptr(), rows, cols)
        ref.gpu_sync()
        scaled("c4", "row softmax", host(sm), host(r), "reference kernel")
        ref.gpu_layernorm(xd.data_ptr(), r.data_ptr(), rows, cols)
        ref.gpu_sync()
        scaled("c4", "layernorm", host(ln), host(r), "reference kernel")
    for name, k, allowed in (("gelu", 2, 2), ("sigmoid", 3, 2), ("tanh", 4, 3)):
        part = x[:8192]
        pd = dev(part)
        got = fdl.unary(pd, k)
        transcendental_vs_twin("c4", f"{name} (first 8192 rows)", part, host(got), orc.unary(part, k).reshape(part.shape))
        if have_ref:
            r = torch.empty_like(pd)
            ref.gpu_activation(pd.data_ptr(), r.data_ptr(), part.size, k, 0.01)
            ref.gpu_sync()
            ulps("c4", f"{name} (first 8192 rows)", host(got), host(r), 2, "reference kernel")


def c5(have_ref):
    n = 1 << 28
    x = np.random.default_rng(42).uniform(-1, 1, n).astype(np.float32)
    y = np.random.default_rng(43).uniform(-1, 1, n).astype(np.float32)
    row = np.random.default_rng(44).uniform(-1, 1, (1, 16384)).astype(np.float32)
    xd, yd, rd = dev(x), dev(y), dev(row)
    z = fdl.binary(xd, yd, fdl.ADD)
    exact("c5", "x + y", host(z), orc.binary(x, y, fdl.ADD))
    if have_ref:
        r = torch.empty_like(xd)
        ref.gpu_vector_add(xd.data_ptr(), yd.data_ptr(), r.data_ptr(), n)
        ref.gpu_sync()
        exact("c5", "x + y", host(z), host(r), "reference kernel (vector_add)")
        exact("c5", "x + y", host(z), ref.cpu_vector_add(x, y, threads=ref.hardware_threads()),
              "reference CPU function")
        del r
    del z
    w = fdl.broadcast_binary(xd.reshape(16384, 16384), rd, fdl.ADD)
    exact("c5", "view[16384,16384] + row[1,16384]", host(w), x.reshape(16384, 16384) + row)
    del w
    s32, s64 = fdl.full_sum(xd, want_f64=True)
    truth = orc.full_sum(x)
    norm = orc.norm2(x)
    sums("c5", "full sum (fp32 result)", host(s32)[0], truth, norm)
    sums("c5", "full sum (f64 result)", host(s64)[0], truth, norm)
    record("c5", "full sum, run twice", "itself", "differing elements",
           differing(host(fdl.full_sum(xd)), host(fdl.full_sum(xd))), 0)


CONFIGS = {"c1": c1, "c2": c2, "c3": c3, "c4": c4, "c5": c5}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="c1,c2,c3,c4,c5")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    build.build_kernels()
    torch.cuda.set_device(0)
    fdl.use_device(0)
    have_ref = ref.available()
    if have_ref:
        ref.gpu_set_device(0)
    for name in args.configs.split(","):
        CONFIGS[name](have_ref)
        torch.cuda.synchronize()
        fdl.take_device_error()
        torch.cuda.empty_cache()
    lines = ["| config | op | against | figure | value | allowed | ok |", "|---|---|---|---|---|---|---|"]
    for config, op, against, form, figure, allowed, ok in ROWS:
        shown = str(figure) if isinstance(figure, int) else f"{figure:.3e}"
        limit = "-" if allowed == INFO else f"{allowed:g}"
        lines.append(f"| {config} | {op} | {against} | {form} | {shown} | {limit} | {'yes' if ok else 'NO'} |")
    text = "\n".join(lines)
    print(text)
    if args.out:
        Path(args.out).write_text(text + "\n")
    if FAILED:
        print("OUTSIDE ALLOWANCE:", FAILED, file=sys.stderr)
        sys.exit(1)


if __name__ == "__main__":
    main()
