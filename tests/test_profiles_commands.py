"""The ncu summaries under profiles/ each give the command that made them; those commands must
keep running committed files with options that exist: every `python bench.py ...` line found
there is parsed against the option list bench.py itself declares (nothing is executed)."""
import glob
import os
import re
import shlex

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, ".."))


def _bench_options():
    src = open(os.path.join(ROOT, "bench.py")).read()
    opts = {}
    for m in re.finditer(r'add_argument\("(--[a-z0-9-]+)"([^\n]*)', src):
        rest = m.group(2)
        choices = re.search(r"choices=\[([^\]]*)\]", rest)
        opts[m.group(1)] = {"flag": "store_true" in rest or "store_false" in rest,
                            "choices": [c.strip(" \"'") for c in choices.group(1).split(",")] if choices else None}
    return opts


def test_profile_commands_use_options_bench_has():
    opts = _bench_options()
    assert "--workload" in opts and "--only-layers" in opts and opts["--no-e2e"]["flag"]
    files = sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md")))
    assert len(files) >= 30
    seen = 0
    for path in files:
        text = open(path).read()
        assert "ncu" in text and "--clock-control none" in text, os.path.basename(path)
        for line in text.splitlines():
            line = line.strip().rstrip("\\").strip()
            if not line.startswith("python bench.py"):
                continue
            # placeholders of the summaries that cover several launches: "{0,7}", "L", "[--ablate ...]", "..."
            line = re.sub(r"\[[^\]]*\]|\([^)]*\)|\.\.\.", " ", line)
            toks = shlex.split(line)[2:]
            i = 0
            while i < len(toks):
                t = toks[i]
                assert t.startswith("--"), (os.path.basename(path), line)
                assert t in opts, "%s: bench.py has no option %s" % (os.path.basename(path), t)
                if opts[t]["flag"]:
                    i += 1
                    continue
                assert i + 1 < len(toks), (os.path.basename(path), line)
                val = toks[i + 1]
                if opts[t]["choices"] and not re.search(r"[{}|]", val):
                    assert val in opts[t]["choices"], "%s: %s %s" % (os.path.basename(path), t, val)
                i += 2
            seen += 1
    assert seen >= 30


def test_every_profile_is_named_for_a_kernel_or_workload_and_not_for_a_round():
    for path in glob.glob(os.path.join(ROOT, "profiles", "*")):
        name = os.path.basename(path)
        assert name.endswith((".md", ".txt")), name + ": profiles/ holds text summaries only"
        assert not re.search(r"(^|_)r(ound)?_?\d+(_|\.|$)", name), name
        assert os.path.getsize(path) < 16 * 1024, name + " is larger than a summary should be"
