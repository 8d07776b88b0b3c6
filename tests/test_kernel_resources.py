"""What ptxas made of the kernels (registers, spills), read from the build log: the kernels on the hot
path must not spill.  A second loop body added to the backward kernel once cost its main loop 800 bytes of
spills and 40 % of its throughput without failing any parity test; this pins that."""
import re

from cgadimpl_b200 import build


def _demangled_like(name):
    """(kernel, template argument list) from a mangled name, e.g. ('rmsnorm_bwd_staged', ['f', '8', '1', '1', '512', '1', '0'])."""
    m = re.match(r"_ZN3agb\d+([a-z_0-9]+?)I(.*)EEv", name)
    if not m:
        return None, []
    out = []
    for tok in re.finditer(r"13__nv_bfloat16|f|Li\d+E|Lb[01]E", m.group(2)):
        t = tok.group(0)
        out.append("bf16" if t.startswith("13") else "f32" if t == "f" else t[2:-1])
    return m.group(1), out


def test_hot_path_kernels_do_not_spill():
    res = build.kernel_resources()
    assert res, "no ptxas log"
    checked = 0
    for name, r in res.items():
        kernel, args = _demangled_like(name)
        hot = False
        if kernel == "rmsnorm_bwd_staged" and len(args) == 7:
            # <T, VPT, HAS_GAMMA, FULL, MAXT, POW2, MULTI>: the 32-elements-per-thread form, every row a full tiling
            hot = args[4] == "512" and args[3] == "1" and args[6] == "0"
        elif kernel == "rmsnorm_fwd_staged" and len(args) == 5:
            # <T, VPT, HAS_GAMMA, FUSE_ADD, FULL>: four vectors per thread, full tiling, without the fused add
            hot = args[1] == "4" and args[4] == "1" and args[3] == "0"
        elif kernel in ("softmax_bwd_staged", "rmsnorm_jvp_staged", "layernorm_jvp_staged"):
            hot = True
        elif kernel == "rmsnorm_bwd_fast" and len(args) == 7:
            # <T, VPT, HAS_GAMMA, FULL, MAXT, KEEP, REL>: the fp32-accumulating 16-bit backward in all its register
            # budgets (80 registers at 768 threads, 102 at 640, 128 at 512, 168 at 384, 255 at 256), with gamma
            hot = args[2] == "1"
            if hot:
                checked += 1
                assert r.get("spill_stores", 0) == 0 and r.get("spill_loads", 0) == 0, f"{name} spills: {r}"
                assert r.get("registers", 0) <= {"768": 80, "640": 102, "512": 128, "384": 168, "256": 255}[args[4]], f"{name}: {r}"
            continue
        elif kernel == "rmsnorm_fwd_fast" and len(args) == 6:
            # <T, VPT, HAS_GAMMA, FUSE_ADD, FULL, FREE>: four vectors per thread with gamma; a register or two
            # parked in local memory outside the vector loops is tolerated, a spilled loop is not
            if args[1] == "4" and args[2] == "1":
                checked += 1
                assert r.get("spill_stores", 0) <= 16 and r.get("spill_loads", 0) <= 16, f"{name} spills: {r}"
            continue
        if hot:
            checked += 1
            assert r.get("spill_stores", 0) == 0 and r.get("spill_loads", 0) == 0, f"{name} spills: {r}"
            assert r.get("registers", 0) <= 128, f"{name}: {r}"
    assert checked >= 26, f"only {checked} hot kernels found in the ptxas log"
