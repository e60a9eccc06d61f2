"""Repository gates run as tests (the reference keeps these as shell gates, scripts/gates/*.sh): every
environment switch the code reads is documented, no machine paths in the sources, every profile
summary states its command, every native source is compiled by the build entry point."""
import re
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
SRC_EXT = {".py", ".cu", ".cuh", ".cpp", ".h", ".hpp"}


def _tracked():
    out = subprocess.run(["git", "ls-files"], cwd=ROOT, capture_output=True, text=True)
    if out.returncode != 0 or not out.stdout.strip():
        files = [p.relative_to(ROOT) for p in ROOT.rglob("*") if p.is_file()]
        skip = ("_work", "gpurun_out", "baseline", ".git", "build")
        return [p for p in files if p.parts[0] not in skip]
    return [Path(l) for l in out.stdout.splitlines()]


def _sources():
    return [p for p in _tracked() if p.suffix in SRC_EXT and (ROOT / p).exists()]


def test_every_environment_switch_is_documented():
    readme = (ROOT / "README.md").read_text()
    pat = re.compile(r"(?:getenv\(|environ(?:\.get)?[\(\[])\s*\"((?:BRAIN|BB)_[A-Z0-9_]+)\"")
    seen = set()
    for p in _sources():
        if p.parts[0] == "tests":
            continue
        seen |= set(pat.findall((ROOT / p).read_text(errors="replace")))
    assert seen, "the scan found no environment reads at all"
    missing = sorted(v for v in seen if v not in readme)
    assert not missing, f"undocumented environment switches: {missing}"


def test_no_machine_paths_in_sources():
    bad = []
    pat = re.compile(r"(/root/|/home/[a-z]|/Users/)")
    for p in _sources():
        if p.name == "test_repo_hygiene.py":
            continue
        for i, line in enumerate((ROOT / p).read_text(errors="replace").splitlines(), 1):
            if pat.search(line):
                bad.append(f"{p}:{i}")
    assert not bad, bad


def test_profile_summaries_state_their_command():
    files = sorted((ROOT / "profiles").glob("*"))
    assert files
    for f in files:
        assert f.suffix in (".md", ".txt"), f"{f.name}: profiles/ holds text summaries only"
        text = f.read_text()
        assert re.search(r"(?im)^\s*(command|commands)\b|`(python|ncu|torchrun) ", text), f"{f.name}: no command"
        assert not re.search(r"(?i)\bround[ _-]?\d", f.name), f.name
        assert "_work/" not in text, f"{f.name}: names a scratch file"


def test_every_native_source_is_built_by_the_entry_point():
    """A .cu / .cpp file under csrc/ that no build list names would silently never be compiled."""
    build_text = "".join((ROOT / p).read_text() for p in ("__graft_entry__.py", "brain_b200/ops/build.py")
                         if (ROOT / p).exists())
    for extra in ("brain_b200/runtime/_host.py", "brain_b200/ops/_cuda.py", "setup.py"):
        if (ROOT / extra).exists():
            build_text += (ROOT / extra).read_text()
    srcs = [p for p in _tracked() if p.parts[0] == "csrc" and p.suffix in (".cu", ".cpp")]
    assert srcs
    globbed = "glob" in build_text
    for p in srcs:
        assert globbed or p.name in build_text, f"{p} is not in any build list"


def test_arch_ids_used_by_the_cli_are_registered():
    """Every architecture id the CLI dispatches on by name is a row of the architecture table, and
    every built row lists at least one verb."""
    from brain_b200 import arch
    ids = {a.id for a in arch.all_archs()}
    text = (ROOT / "brain_b200/cli/main.py").read_text()
    used = set(re.findall(r"a\.id == \"([a-z0-9]+)\"", text))
    assert used and used <= ids, used - ids
    for a in arch.all_archs(built_only=True):
        assert a.verbs, a.id
        assert arch.by_id(a.id) is a and all(arch.by_id(al) is a for al in a.aliases)
