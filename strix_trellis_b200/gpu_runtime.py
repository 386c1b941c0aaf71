"""Fixture-driven check of the runtime on the GPU, with the coverage of the reference's
`gpu_runtime` executable (reference `docs/GPU_TESTS.md:70-124`):

    python -m strix_trellis_b200.gpu_runtime [--route all|gemv|gemm|grouped|stages|moe] fixture.stgpu | directory [...]

Every number the checks compare against comes from the fixture file (written by the
reference's CPU contract); alpha and beta are applied to it here in binary32 with a separate
multiplication and addition.  Any API, format, stage or tolerance failure gives a nonzero
exit status.  STRANK01 projection files are accepted too (route gemv / gemm only: they carry
no stage checkpoints) and are held to their own per-output bound as well.  A DIRECTORY holding
the six `expert-{gate,up,down}-k{2,3}.strank` files and `moe-*.strank` windows of the reference's
rank generator is run as routed-expert blocks (route moe).
"""
from __future__ import annotations

import argparse
import ctypes as C
import sys

import numpy as np
import torch

from . import native as N
from pathlib import Path

from .fixtures import GpuFixture, RankFixture, RouteWindowFixture, read_fixture, read_strank
from .runtime import Context, MoePlan, _cur_stream

ALPHA_BETA = ((1.0, 0.0), (-0.75, 0.25), (0.0, -0.5), (1.0, -0.0))
GEMV_ROWS = tuple(range(0, 9))
GEMM_ROWS = tuple(range(0, 9)) + (16, 17, 32, 64, 65, 128, 129, 256)
GROUP_ROWS = (1, 2, 0, 4, 8, 16)  # disjoint contiguous slices and one empty group
MAXABS, NRMSE = 5e-4, 3e-5       # reference docs/GPU_TESTS.md:126-131


def expected(ref, old, alpha, beta):
    out = (np.float32(alpha) * ref).astype(np.float32)
    if beta != 0.0:
        out = (out + (np.float32(beta) * old).astype(np.float32)).astype(np.float32)
    return out


class Report:
    def __init__(self, out=sys.stdout):
        self.failures, self.checks, self.out = 0, 0, out

    def line(self, ok, text):
        self.checks += 1
        self.failures += 0 if ok else 1
        print(("PASS " if ok else "FAIL ") + text, file=self.out)

    def tolerance(self, what, actual, reference, bound=None):
        actual, reference = np.asarray(actual, np.float32), np.asarray(reference, np.float32)
        if actual.size == 0:
            return self.line(actual.shape == reference.shape, f"{what} (empty)")
        finite = bool(np.isfinite(actual).all())
        diff = np.abs(actual.astype(np.float64) - reference.astype(np.float64))
        worst = int(np.argmax(diff)) if finite else int(np.argmax(~np.isfinite(actual)))
        maxabs, maxref = float(diff.max()) if finite else float("inf"), float(np.abs(reference).max())
        nrmse = float(np.sqrt((diff ** 2).sum() / max(float((reference.astype(np.float64) ** 2).sum()), 1e-30))) \
            if finite else float("inf")
        ok = finite and maxabs <= MAXABS * max(1.0, maxref) and nrmse <= NRMSE
        if ok and bound is not None:
            ok = bool((diff <= bound).all())
        self.line(ok, f"{what} maxabs={maxabs:.3e} maxref={maxref:.3e} nrmse={nrmse:.3e} worst={worst}")

    def identical(self, what, actual, reference):
        a, b = np.ascontiguousarray(actual), np.ascontiguousarray(reference)
        same = a.shape == b.shape and a.dtype == b.dtype and a.tobytes() == b.tobytes()
        where = ""
        if not same and a.shape == b.shape:
            bad = np.flatnonzero(a.view(np.uint8).reshape(-1) != b.view(np.uint8).reshape(-1))
            where = f" first differing byte {int(bad[0])} of {a.nbytes}"
        self.line(same, f"{what} bytes identical{'' if same else ' NO'}{where}")


def _dev(a):
    return torch.from_numpy(np.array(a, order="C")).cuda()  # a writable copy: sections are read-only views


def _fresh(shape, nan):
    """Output memory for beta == 0: newly allocated, or filled with NaN."""
    y = torch.empty(shape, dtype=torch.float32, device="cuda")
    if nan and y.numel():
        y.fill_(float("nan"))
    return y


def route_stages(rep, ctx, fx: GpuFixture, w):
    tag = f"{fx.name} stages"
    rep.identical(f"{tag} Q[{fx.meta.inputs},{fx.meta.outputs}]", w.dequantize().cpu().numpy().view(np.uint16),
                  fx.q.view(np.uint16))
    scaled, inh, a = w.input_stages(_dev(fx.x))
    rep.identical(f"{tag} scaled f16", scaled.cpu().numpy().view(np.uint16), fx.scaled.view(np.uint16))
    rep.identical(f"{tag} input H128 f32", inh.cpu().numpy().view(np.uint32), fx.inh.view(np.uint32))
    rep.identical(f"{tag} core input f16", a.cpu().numpy().view(np.uint16), fx.a.view(np.uint16))
    rep.identical(f"{tag} ordered core f32", w.core_exact(_dev(fx.a)).cpu().numpy().view(np.uint32),
                  fx.core.view(np.uint32))
    for alpha, beta in ALPHA_BETA:
        y = _dev(fx.old) if beta != 0.0 else _fresh(fx.ref.shape, nan=True)
        got = w.output_stages(_dev(fx.core), alpha, beta, y).cpu().numpy()
        rep.tolerance(f"{tag} output stages alpha={alpha} beta={beta}", got, expected(fx.ref, fx.old, alpha, beta))


def _matmul(rep, fx, w, call, route, rows_list):
    cap = fx.meta.rows
    bound = getattr(fx, "bound", None)
    for rows in (r for r in rows_list if r <= cap):
        ranks = (1, 2) if (rows == 1 and route == "gemv") else (2,)
        for rank in ranks:
            for alpha, beta in ALPHA_BETA:
                for nan in ((False, True) if beta == 0.0 else (False,)):
                    x = _dev(fx.x[:rows]) if rows else torch.empty((0, fx.meta.inputs), device="cuda")
                    if beta != 0.0:
                        y = _dev(fx.old[:rows]) if rows else torch.empty((0, fx.meta.outputs), device="cuda")
                    else:
                        y = _fresh((rows, fx.meta.outputs), nan)
                    if rank == 1:
                        x, y = x[0], y[0]
                    if rows == 0:  # validates, launches nothing, needs no workspace
                        need = w.workspace_bytes(x, y)
                        call(x, y, alpha, beta)
                        rep.line(need == 0, f"{fx.name} {route} rows=0 rank={rank} workspace={need}")
                        continue
                    got = call(x, y, alpha, beta).cpu().numpy().reshape(rows, -1)
                    want = expected(fx.ref[:rows], fx.old[:rows], alpha, beta)
                    lim = None
                    if bound is not None:
                        lim = abs(alpha) * bound[:rows] + 4 * 2.0 ** -24 * (np.abs(want) + abs(beta) * np.abs(fx.old[:rows]))
                    rep.tolerance(f"{fx.name} {route} rows={rows} rank={rank} alpha={alpha} beta={beta}"
                                  f"{' nan-filled' if nan else ''}", got, want, lim)


def route_gemv(rep, ctx, fx, w):
    _matmul(rep, fx, w, lambda x, y, a, b: w.gemv(x, y, a, b), "gemv", GEMV_ROWS)


def route_gemm(rep, ctx, fx, w):
    _matmul(rep, fx, w, lambda x, y, a, b: w.gemm(x, y, a, b), "gemm", GEMM_ROWS)


def _grouped_call(ctx, descs):
    lib = ctx.lib
    groups = (N.MatmulDesc * len(descs))(*descs)
    d = N.GroupedMoeDesc()
    d.struct_size, d.abi_version = C.sizeof(N.GroupedMoeDesc), N.ABI_VERSION
    d.groups, d.group_count = groups, len(descs)
    need = N.u64(0)
    N.check(lib.strix_grouped_moe_workspace_bytes(ctx.handle, C.byref(d), C.byref(need)), "grouped workspace")
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda")
    d.workspace, d.workspace_bytes = (ws.data_ptr(), need.value) if need.value else (None, 0)
    sd = _cur_stream()
    N.check(lib.strix_grouped_moe(ctx.handle, C.byref(d), C.byref(sd)), "strix_grouped_moe")
    torch.cuda.synchronize()
    return ws


def route_grouped(rep, ctx, fx: GpuFixture, w):
    """Disjoint contiguous row slices as groups of one call, alternating between the
    fixture's expert and a second expert whose svh is zero (its reference is pure bias):
    a handle that is ignored shows at once."""
    class Muted:
        trellis, suh, bias, bits, codebook = fx.trellis, fx.suh, fx.bias, fx.bits, fx.codebook
        svh = np.zeros_like(fx.svh)
    muted = ctx.prepare(Muted)
    pure_bias = np.broadcast_to(fx.bias if fx.bias is not None else np.zeros(fx.meta.outputs, np.float32),
                                fx.ref.shape)
    for alpha, beta in ALPHA_BETA:
        at, xs, ys, descs, wants, owners = 0, [], [], [], [], []
        for g, rows in enumerate(r for r in GROUP_ROWS):
            rows = min(rows, fx.meta.rows - at)
            owner, ref = (w, fx.ref) if g % 2 == 0 else (muted, pure_bias)
            x = _dev(fx.x[at:at + rows]) if rows else torch.empty((0, fx.meta.inputs), device="cuda")
            y = (_dev(fx.old[at:at + rows]) if beta != 0.0 else _fresh((rows, fx.meta.outputs), True)) if rows \
                else torch.empty((0, fx.meta.outputs), device="cuda")
            xs.append(x), ys.append(y), owners.append(owner)
            descs.append(owner.matmul_desc(x, y, alpha, beta))
            wants.append(expected(ref[at:at + rows], fx.old[at:at + rows], alpha, beta))
            at += rows
        keep = _grouped_call(ctx, descs)
        for g, (y, want) in enumerate(zip(ys, wants)):
            rep.tolerance(f"{fx.name} grouped group={g} rows={len(want)} alpha={alpha} beta={beta}",
                          y.cpu().numpy(), want)
        # each group alone through the same route
        for g, (x, want) in enumerate(zip(xs, wants)):
            if not len(want):
                continue
            rows = len(want)
            lo = sum(len(t) for t in wants[:g])
            y1 = _dev(fx.old[lo:lo + rows]) if beta != 0.0 else _fresh((rows, fx.meta.outputs), True)
            keep1 = _grouped_call(ctx, [owners[g].matmul_desc(x, y1, alpha, beta)])
            rep.identical(f"{fx.name} grouped group={g} alone vs in the batch alpha={alpha} beta={beta}",
                          y1.cpu().numpy(), ys[g].cpu().numpy())
            del keep1
        del keep
    muted.close()


# ---- routed-expert windows ------------------------------------------------------------
# How the reference's generator derives a bank of experts from its six projection files
# (tools/make_rank_fixtures.py:127-145): bank id = 17 + 3*index; the rate of each projection
# and a per-expert bias offset depend on the index.
MOE_NRMSE = 1e-4  # three chained projections with a binary16 rounding between them


def _expert_index(expert_id):
    return (int(expert_id) - 17) // 3


def _expert_bits(index, projection):
    if projection == "gate":
        return 2 + index % 2
    if projection == "up":
        return 3 if index % 3 == 0 else 2
    return 2 if index % 3 == 1 else 3


def _expert_bias(base, index, projection):
    factor = {"gate": 1.0, "up": -0.5, "down": 0.25}[projection]
    return (base.astype(np.float32) + np.float32((17 + 3 * index + 1) * factor / 512)).astype(np.float32)


def route_moe(rep, ctx, directory):
    directory = Path(directory)
    files = {(p, k): read_strank(directory / f"expert-{p}-k{k}.strank")
             for p in ("gate", "up", "down") for k in (2, 3)}
    x = files[("gate", 2)].x  # gate and up projections share one input
    windows = sorted(directory.glob("moe-*.strank"))
    rep.line(bool(windows), f"{directory.name}: {len(windows)} routed-expert windows")
    for path in windows:
        fx = read_strank(path)
        if not isinstance(fx, RouteWindowFixture):
            rep.line(False, f"{path.name}: not a routed-expert window")
            continue
        ids = np.unique(fx.routes)
        experts = []
        for eid in ids:
            index, triple = _expert_index(eid), []
            for projection in ("gate", "up", "down"):
                f = files[(projection, _expert_bits(index, projection))]

                class Layer:
                    trellis, suh, svh, bits, codebook = f.trellis, f.suh, f.svh, f.bits, f.codebook
                    bias = _expert_bias(f.bias, index, projection)
                triple.append(ctx.prepare(Layer))
            experts.append(tuple(triple))
        rows = fx.meta.rows
        for alpha, beta in ALPHA_BETA:
            y = _dev(fx.old) if beta != 0.0 else _fresh(fx.ref.shape, nan=True)
            plan = MoePlan(ctx, experts, _dev(x[:rows]), y, fx.routes, fx.scores, expert_ids=ids, alpha=alpha, beta=beta)
            plan.submit()
            torch.cuda.synchronize()
            got, hidden = y.cpu().numpy(), plan.hidden().cpu().numpy()
            plan.close()
            want = expected(fx.ref, fx.old, alpha, beta)
            diff = np.abs(got.astype(np.float64) - want)
            finite = bool(np.isfinite(got).all())
            nrmse = float(np.sqrt((diff ** 2).sum() / max(float((want.astype(np.float64) ** 2).sum()), 1e-30)))
            ok = finite and diff.max() <= MAXABS * max(1.0, float(np.abs(want).max())) and nrmse <= MOE_NRMSE
            rep.line(ok, f"{fx.name} block experts={len(ids)} alpha={alpha} beta={beta} maxabs={diff.max():.3e} "
                         f"maxref={np.abs(want).max():.3e} nrmse={nrmse:.3e}")
        live = fx.scores != 0  # a zero score skips its slot: nothing is written there
        rep.tolerance(f"{fx.name} SwiGLU values of the scored slots", hidden[live], fx.hidden[live])
        for triple in experts:
            for w in triple:
                w.close()


ROUTES = {"stages": route_stages, "gemv": route_gemv, "gemm": route_gemm, "grouped": route_grouped}


def run(paths, route="all", out=sys.stdout):
    """Run the requested routes over the fixture files; returns the number of failed checks."""
    rep = Report(out)
    ctx = Context(0)
    props = torch.cuda.get_device_properties(0)
    print(f"device 0: {props.name}, sm_{props.major}{props.minor}, {props.multi_processor_count} SMs, warp 32",
          file=out)
    stream = torch.cuda.Stream()  # explicit non-blocking stream for uploads, launches and downloads
    with torch.cuda.stream(stream):
        for path in paths:
            if Path(path).is_dir():
                if route in ("all", "moe"):
                    route_moe(rep, ctx, path)
                continue
            if route == "moe":
                rep.line(False, f"{path}: route moe takes a directory")
                continue
            fx = read_fixture(path)
            if not isinstance(fx, (GpuFixture, RankFixture)):
                rep.line(False, f"{path}: routed-expert windows are not a matmul fixture")
                continue
            names = list(ROUTES) if route == "all" else [route]
            if isinstance(fx, RankFixture):
                names = [n for n in names if n in ("gemv", "gemm")]
            w = ctx.prepare(fx, use_blob=True)
            for name in names:
                ROUTES[name](rep, ctx, fx, w)
            stream.synchronize()
            w.close()
        rep.line(ctx.device_status() == 0, "device status word clear")
    ctx.close()
    print(f"{rep.checks - rep.failures} of {rep.checks} checks passed", file=out)
    return rep.failures


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--route", choices=["all", *ROUTES, "moe"], default="all")
    p.add_argument("fixtures", nargs="+")
    a = p.parse_args(argv)
    return 1 if run(a.fixtures, a.route) else 0


if __name__ == "__main__":
    sys.exit(main())
