"""Source-level rules of this code base, checked over every tracked source file:

* no TMA / bulk load with cluster multicast anywhere (a load whose source could be another GPU's memory must never carry
  it, and the multi-GPU entry points share their kernels with the single-GPU ones);
* none of the batched memcpy runtime calls (one ``cudaMemcpyAsync`` per copy, or a gather kernel, instead);
* every ``ncu`` command quoted in the summaries under ``profiles/`` keeps the clocks alone;
* no kernel spins without a bound: every ``while`` / ``do`` loop that polls an mbarrier or a peer counter sits next to a
  cycle limit.
"""
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC_EXT = (".cu", ".cuh", ".h", ".cpp", ".inl", ".py")


def _sources():
    out = []
    for base in ("hippolm_b200", "bench", "scripts", "baseline"):
        for dp, dn, fn in os.walk(os.path.join(ROOT, base)):
            if os.sep + "_ref" in dp or "__pycache__" in dp or os.sep + "lib" + os.sep in dp + os.sep:
                continue
            out += [os.path.join(dp, f) for f in fn if f.endswith(SRC_EXT)]
    out += [os.path.join(ROOT, f) for f in ("bench.py", "__graft_entry__.py")]
    return out


def test_no_cluster_multicast_loads_and_no_batched_memcpy():
    multicast = "multicast" + "::" + "cluster"
    batched = ["cuda" + "Memcpy" + "BatchAsync", "cuda" + "Memcpy3D" + "BatchAsync", "cu" + "Memcpy" + "BatchAsync",
               "cu" + "Memcpy3D" + "BatchAsync"]
    for p in _sources():
        text = open(p, errors="replace").read()
        for m in re.finditer(re.escape(multicast), text):
            line = text[text.rfind("\n", 0, m.start()) + 1:text.find("\n", m.end())]
            # the only form that is open on any number of GPUs is the commit of the tensor-core pipeline
            assert "tcgen05.commit" in line, f"{p}: cluster multicast outside tcgen05.commit: {line.strip()}"
        for b in batched:
            assert b not in text, f"{p} names {b}"


def test_profile_commands_leave_the_clocks_alone():
    for p in glob.glob(os.path.join(ROOT, "profiles", "*.md")):
        text = open(p).read().replace("\\\n", " ")
        for line in text.splitlines():
            s = line.strip()
            if re.match(r"^(\S+=\S+\s+)*ncu\s", s) or re.search(r"&&\s*ncu\s", s):
                if " -i " in s or "--page" in s or "--list-" in s or "--query-metrics" in s:
                    continue                      # reading a report / listing names runs nothing on a GPU
                assert "--clock-control none" in s, f"{p}: {s}"


def test_device_side_waits_are_bounded():
    """Every polling loop in the kernels compares against a limit (clock64 difference or an iteration count) and reports
    through the status word instead of spinning forever."""
    polls = ("mbar_try_wait", "ld_acquire_sys", "ld.acquire.sys")
    for p in glob.glob(os.path.join(ROOT, "hippolm_b200", "csrc", "*.cu*")):
        lines = open(p).read().splitlines()
        for i, l in enumerate(lines):
            if re.search(r"\b(while|do)\b", l) and any(k in " ".join(lines[i:i + 4]) for k in polls):
                window = " ".join(lines[max(0, i - 3):i + 8])
                assert "clock64" in window or "limit" in window or "kWait" in window, f"{p}:{i + 1}: unbounded poll? {l.strip()}"
