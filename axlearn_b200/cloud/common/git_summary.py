"""A snapshot of the submitting checkout's git state (reference: axlearn/cloud/common/git_summary.py:16-254).

Recorded with every bundle so that a running job can be traced back to the code it was built
from: as image labels (short values) and as files inside the bundle (full values, e.g. the
uncommitted diff).
"""

from __future__ import annotations

import dataclasses
import enum
import os
import re
import subprocess
from typing import Optional


@dataclasses.dataclass(frozen=True)
class GitSummaryMember:
    """One fact about the checkout: the git command that yields it and the file it is stored in."""

    cmd: str
    file: str
    label_ok: bool = True          # False: too long / free-form to be a label value

    def execute_command(self, cwd: str) -> str:
        out = subprocess.run(self.cmd.split(), cwd=cwd, capture_output=True, text=True, check=False)
        if out.returncode != 0:
            raise subprocess.CalledProcessError(out.returncode, self.cmd, out.stdout, out.stderr)
        return out.stdout.strip()

    def to_label(self, val: str) -> str:
        """Label values allow ``[a-z0-9_-]`` only and at most 63 characters."""
        return re.sub(r"[^a-z0-9_-]", "_", val.lower())[:63]

    def to_file(self, *, folder: str, val: str) -> str:
        path = os.path.join(folder, self.file)
        with open(path, "w", encoding="utf-8") as f:
            f.write(val)
        return path


class GitSummaryMembers(enum.Enum):
    commit = GitSummaryMember("git rev-parse HEAD", ".git.commit")
    branch = GitSummaryMember("git rev-parse --abbrev-ref HEAD", ".git.branch")
    origin = GitSummaryMember("git remote get-url origin", ".git.origin")
    porcelain = GitSummaryMember("git status --porcelain", ".git.porcelain", label_ok=False)
    diff = GitSummaryMember("git diff HEAD", ".git.diff", label_ok=False)


@dataclasses.dataclass
class GitSummary:
    """Runs every member's command in ``path`` (members whose command fails -- no remote, not a
    checkout -- are left out)."""

    path: str = "."
    required: tuple = (GitSummaryMembers.commit,)
    summary: dict = dataclasses.field(default_factory=dict)

    def __post_init__(self):
        for member in GitSummaryMembers:
            try:
                self.summary[member] = member.value.execute_command(self.path)
            except (subprocess.CalledProcessError, FileNotFoundError, NotADirectoryError):
                continue

    def is_valid(self) -> bool:
        return all(m in self.summary for m in self.required)

    def is_dirty(self) -> bool:
        if not self.is_valid():
            return False
        return bool(self.summary.get(GitSummaryMembers.porcelain))

    def to_labels(self) -> dict[str, str]:
        out = {}
        for member, val in self.summary.items():
            if member.value.label_ok:
                out[f"git-{member.name}"] = member.value.to_label(val)
        return out

    def to_disk(self, out_dir: str) -> list[str]:
        os.makedirs(out_dir, exist_ok=True)
        return [member.value.to_file(folder=out_dir, val=val) for member, val in self.summary.items()]

    def __getitem__(self, key: GitSummaryMembers) -> Optional[str]:
        return self.summary.get(key)

    def __bool__(self) -> bool:
        return self.is_valid()
