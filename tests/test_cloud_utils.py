"""Cloud helper utilities and bastion tables (reference behaviour: axlearn/cloud/common/utils.py,
axlearn/cloud/gcp/jobs/launch_utils.py:123-212)."""

import datetime
import re

import pytest

from axlearn_b200.cloud.common import utils
from axlearn_b200.cloud.common.bastion import BastionJob, JobState, JobStatus
from axlearn_b200.cloud.common.job_types import JobMetadata, JobSpec


def test_small_helpers():
    assert re.fullmatch(r"[a-z0-9-]+-[0-9a-f]{5}", utils.generate_job_name())
    assert utils.generate_job_id() != utils.generate_job_id()
    assert utils.parse_kv_flags(["a:1", "b:x:y", "a:2"]) == {"a": "2", "b": "x:y"}
    assert utils.parse_kv_flags(["a=1"], delimiter="=") == {"a": "1"}
    with pytest.raises(ValueError):
        utils.parse_kv_flags(["a"])
    assert utils.canonicalize_to_list("a, b,c") == ["a", "b", "c"] and utils.canonicalize_to_list("") == []
    assert utils.canonicalize_to_list(["a", "b"]) == ["a", "b"]
    assert utils.canonicalize_to_string(["a ", "b"]) == "a,b" and utils.canonicalize_to_string(None) == ""
    assert utils.parse_action(["cli", "--flag", "start", "x"], options=["start", "stop"]) == "start"
    assert utils.parse_action(["cli", "bogus"], options=["start", "stop"], default="stop") == "stop"
    with pytest.raises(ValueError):
        utils.parse_action(["cli"], options=["start"])
    base = {"a": {"b": 1, "c": 2}, "d": 3}
    assert utils.merge(base, {"a": {"b": 5, "e": {"f": 1}}, "d": {"g": 1}}) == {"a": {"b": 5, "c": 2, "e": {"f": 1}}, "d": {"g": 1}}
    assert utils.to_bool("True") is True and utils.to_bool("false") is False and utils.to_bool(True) is True
    with pytest.raises(ValueError):
        utils.to_bool("1")


def test_table():
    t = utils.Table(headings=["a", "b"], rows=[[1, 2], [3, 4]])
    t.add_row([5, 6])
    t.add_col("c", ["x", "y", "z"])
    assert t.get_col("c", "a") == [["x", 1], ["y", 3], ["z", 5]]
    t.sort(key=lambda r: r[0], reverse=True)
    assert t.rows[0] == [5, 6, "z"]
    with pytest.raises(ValueError):
        t.add_row([1])
    with pytest.raises(ValueError):
        t.add_col("d", [1])
    text = repr(t)
    assert text.splitlines()[1].split() == ["A", "B", "C"] and text.splitlines()[2].split() == ["5", "6", "z"]
    assert t == utils.Table(headings=["a", "b", "c"], rows=[[5, 6, "z"], [3, 4, "y"], [1, 2, "x"]])
    empty = utils.Table(headings=[], rows=[])
    empty.add_col("k", [1, 2])
    assert empty.rows == [[1], [2]]


def _job(name, user, project, state, resources, tier=None):
    meta = JobMetadata(user_id=user, project_id=project, creation_time=datetime.datetime(2024, 1, 1), resources=resources,
                       priority=3, job_id=f"id-{name}")
    spec = JobSpec(version=1, name=name, command="true", cleanup_command=None, env_vars=None, metadata=meta)
    return BastionJob(spec=spec, state=JobStatus(state, metadata={} if tier is None else {"tier": tier}))


def test_job_and_usage_tables():
    jobs = {"a": _job("a", "ann", "p1", JobState.ACTIVE, {"b200": 8}, tier=0),
            "b": _job("b", "bob", "p1", JobState.ACTIVE, {"b200": 16, "cpu": 4}, tier=1),
            "c": _job("c", "ann", "p2", JobState.PENDING, {"b200": 64}),
            "d": _job("d", "ann", "p2", JobState.CLEANING, {"b200": 8})}
    t = utils.jobs_table(jobs)
    assert t.headings[0] == "NAME" and t.get_col("NAME", "JOB_STATE", "TIER")[2] == ["c", "PENDING", "None"]
    assert t.get_col("RESOURCES")[1] == ["{'b200': 16, 'cpu': 4}"]
    by_user = utils.user_usage_table(jobs)
    assert by_user.rows == [["bob", "cpu", 4, 1], ["ann", "b200", 16, 2], ["bob", "b200", 16, 1]]
    by_project = utils.project_usage_table(jobs)
    assert by_project.rows == [["p1", "cpu", 4, 1], ["p1", "b200", 24, 2], ["p2", "b200", 8, 1]]


def test_bastion_list_table(tmp_path, capsys):
    from axlearn_b200.cli.main import main

    root = str(tmp_path / "bastion")
    assert main(["bastion", "submit", "--root_dir", root, "--name", "j1", "--command", "true", "--user", "ann",
                 "--project", "p", "--resources", "b200=8"]) == 0
    capsys.readouterr()
    assert main(["bastion", "list", "--root_dir", root, "--format", "table"]) == 0
    out = capsys.readouterr().out
    assert "NAME" in out and "j1" in out and "PENDING" in out and "Usage by project:" in out
