"""Docker / tar / GCP bundlers, git summary, uploader, writer, validators, mutators -- all against
recording runners and temporary directories."""

import datetime
import os
import subprocess
import tarfile
import time
import types

import pytest

from axlearn_b200.cloud.common import docker
from axlearn_b200.cloud.common.bundler import DockerBundler, get_bundler_config
from axlearn_b200.cloud.common.git_summary import GitSummary, GitSummaryMembers
from axlearn_b200.cloud.common.job_types import JobMetadata, JobSpec
from axlearn_b200.cloud.common.pod_mutator import MergePodMutator, PrefixCommandPatcher
from axlearn_b200.cloud.common.uploader import Uploader, mirror_directory, with_interval
from axlearn_b200.cloud.common.validator import CompositeValidator, ResourceLimitValidator, ValidationError
from axlearn_b200.cloud.common.writer import FileWriter
from axlearn_b200.cloud.gcp.bundler import CloudBuildBundler, GCSTarBundler, region_from_worker_pool


def _git(cwd, *args):
    subprocess.run(["git", *args], cwd=cwd, check=True, capture_output=True,
                   env={**os.environ, "GIT_AUTHOR_NAME": "t", "GIT_AUTHOR_EMAIL": "t@t", "GIT_COMMITTER_NAME": "t",
                        "GIT_COMMITTER_EMAIL": "t@t"})


@pytest.fixture
def checkout(tmp_path):
    src = tmp_path / "src"
    (src / "pkg").mkdir(parents=True)
    (src / "pkg" / "a.py").write_text("A = 1\n")
    (src / "pkg" / "a.pyc").write_text("junk")
    (src / "_work").mkdir()
    (src / "_work" / "notes.txt").write_text("scratch")
    (src / "Dockerfile").write_text("FROM scratch\n")
    _git(src, "init", "-q")
    _git(src, "add", "-A")
    _git(src, "commit", "-q", "-m", "init")
    return src


def Recorder(outputs=()):  # pylint: disable=invalid-name
    """A runner that records its argument lists (a plain function: config values must be)."""
    pending = list(outputs)

    def run(args, **kwargs):
        run.calls.append(list(args))
        return types.SimpleNamespace(stdout=pending.pop(0) if pending else "", returncode=0)

    run.calls = []
    return run


def test_git_summary_labels_files_and_dirtiness(checkout, tmp_path):
    s = GitSummary(path=str(checkout))
    assert s.is_valid() and not s.is_dirty()
    assert len(s[GitSummaryMembers.commit]) == 40 and s[GitSummaryMembers.origin] is None
    labels = s.to_labels()
    assert set(labels) == {"git-commit", "git-branch"} and all(len(v) <= 63 for v in labels.values())
    files = s.to_disk(str(tmp_path / "out"))
    assert sorted(os.path.basename(f) for f in files) == [".git.branch", ".git.commit", ".git.diff", ".git.porcelain"]
    (checkout / "pkg" / "a.py").write_text("A = 2\n")
    dirty = GitSummary(path=str(checkout))
    assert dirty.is_dirty() and "A = 2" in dirty[GitSummaryMembers.diff]
    assert not GitSummary(path=str(tmp_path))                      # not a checkout


def test_docker_bundler_builds_sidecars_then_main_and_refuses_dirty_trees(checkout):
    rec = Recorder()
    cfg = get_bundler_config(bundler_type="docker", spec=["image=trainer", "repo=reg.example/proj",
                                                          f"dockerfile={checkout / 'Dockerfile'}"])
    cfg.set(runner=rec, build_args={"extras": ["gpu", "dev"]}, target="main", sidecars=["tee"],
            cache_from=["reg.example/proj/trainer:cache"])
    image = cfg.instantiate().bundle("v1", src_dir=str(checkout))
    assert image == "reg.example/proj/trainer:v1"
    kinds = [(c[1], c[c.index("-t") + 1] if "-t" in c else c[2]) for c in rec.calls]
    assert kinds == [("build", "reg.example/proj/tee:v1"), ("push", "reg.example/proj/tee:v1"),
                     ("build", "reg.example/proj/trainer:v1"), ("push", "reg.example/proj/trainer:v1")]
    main = rec.calls[2]
    assert main[main.index("--target") + 1] == "main" and "extras=gpu,dev" in main and "linux/amd64" in main
    assert any(a.startswith("git-commit=") for a in main) and "--cache-from" in main
    (checkout / "pkg" / "a.py").write_text("A = 3\n")
    with pytest.raises(RuntimeError, match="commit your changes"):
        cfg.instantiate().bundle("v2", src_dir=str(checkout))
    assert cfg.clone(allow_dirty=True).instantiate().bundle("v2", src_dir=str(checkout)).endswith(":v2")
    assert cfg.clone(skip_bundle=True).instantiate().bundle("v3") == "reg.example/proj/trainer:v3"
    with pytest.raises(ValueError):
        DockerBundler.default_config().set(image="", repo="r", dockerfile="d").instantiate()
    assert docker.registry_from_repo("us-docker.pkg.dev/p/r") == "https://us-docker.pkg.dev"


def test_gcs_tar_bundler_packs_the_filtered_tree(checkout, tmp_path):
    seen = {}

    def runner(args, **kwargs):
        assert args[:3] == ["gcloud", "storage", "cp"]
        with tarfile.open(args[3]) as tar:
            seen["names"] = sorted(n[2:] if n.startswith("./") else n for n in tar.getnames() if n != ".")
        seen["dst"] = args[4]
        return types.SimpleNamespace(stdout="")

    b = GCSTarBundler.default_config().set(remote_dir="gs://bucket/jobs", runner=runner).instantiate()
    bundle_id = b.bundle("job1", src_dir=str(checkout))
    assert bundle_id == seen["dst"] == "gs://bucket/jobs/job1/axlearn.tar.gz"
    assert "pkg/a.py" in seen["names"] and ".git.commit" in seen["names"]
    assert not any(n.endswith(".pyc") or n.startswith("_work") or n.startswith(".git/") for n in seen["names"])
    assert b.install_command(bundle_id, dest="/code") == (
        "mkdir -p /code && gcloud storage cp gs://bucket/jobs/job1/axlearn.tar.gz /code/axlearn.tar.gz"
        " && tar -xzf /code/axlearn.tar.gz -C /code")


def test_cloud_build_bundler_submits_and_polls(checkout):
    rec = Recorder(outputs=["build-123\n", "WORKING\n", "SUCCESS\n"])
    pool = "projects/p/locations/us-east5/workerPools/w"
    cfg = CloudBuildBundler.default_config().set(
        image="trainer", repo="us-docker.pkg.dev/p/r", dockerfile=str(checkout / "Dockerfile"), project="p",
        private_worker_pool=pool, poll_seconds=0.0, runner=rec)
    assert cfg.instantiate().bundle("v1", src_dir=str(checkout)) == "us-docker.pkg.dev/p/r/trainer:v1"
    submit, d1, d2 = rec.calls
    assert submit[:3] == ["gcloud", "builds", "submit"] and "--async" in submit
    assert submit[submit.index("--region") + 1] == "us-east5" == region_from_worker_pool(pool)
    assert d1[:4] == ["gcloud", "builds", "describe", "build-123"] and d1 == d2
    built = cfg.instantiate().build_config(dockerfile="/x/Dockerfile", image="i:t", args={"a": "1"}, labels={})
    assert built["images"] == ["i:t"] and built["options"]["pool"] == {"name": pool}
    assert built["steps"][0]["args"][:5] == ["build", "-f", "Dockerfile", "-t", "i:t"]
    kaniko = cfg.clone(use_kaniko=True).instantiate().build_config(dockerfile="/x/Dockerfile", image="i:t", args={},
                                                                    labels={})
    assert kaniko["images"] == [] and "--destination=i:t" in kaniko["steps"][0]["args"]
    failing = Recorder(outputs=["b2\n", "FAILURE\n"])
    with pytest.raises(RuntimeError, match="FAILURE"):
        cfg.clone(runner=failing).instantiate().bundle("v2", src_dir=str(checkout))
    assert region_from_worker_pool("nonsense") is None


def test_uploader_mirrors_until_cleaned_up(tmp_path):
    src, dst = tmp_path / "src", tmp_path / "dst"
    (src / "logs").mkdir(parents=True)
    (src / "logs" / "a.log").write_text("one\n")
    mirror_directory(src_dir=str(src), dst_dir=str(dst))
    assert (dst / "logs" / "a.log").read_text() == "one\n"
    calls = []
    loop = with_interval(lambda **kw: calls.append(kw) or (_ for _ in ()).throw(OSError("flaky")), interval_seconds=0)
    loop(src_dir="s", dst_dir="d", max_rounds=3)                 # failures do not end the loop
    assert len(calls) == 3
    up = Uploader.default_config().set(src_dir=str(src), dst_dir=str(dst),
                                       upload_fn=with_interval(mirror_directory, interval_seconds=0.05)).instantiate()
    up()
    up()                                                           # second call: already running
    (src / "logs" / "b.log").write_text("two\n")
    deadline = time.time() + 10
    while not (dst / "logs" / "b.log").exists() and time.time() < deadline:
        time.sleep(0.05)
    up.cleanup()
    assert (dst / "logs" / "b.log").read_text() == "two\n"


def test_writer_appends_from_a_background_thread(tmp_path):
    path = tmp_path / "out" / "job.log"
    with FileWriter(output_path=str(path), flush_seconds=0.02) as w:
        w.write("a\n")
        time.sleep(0.2)
        assert path.read_text() == "a\n"                          # flushed while still open
        w.write("b\n")
    assert path.read_text() == "a\nb\n"
    with pytest.raises(ValueError):
        w.write("late")


def _job(resources, command="python train.py"):
    meta = JobMetadata(user_id="u", project_id="p", creation_time=datetime.datetime(2024, 1, 1), resources=resources)
    return JobSpec(version=1, name="j", command=command, cleanup_command=None, env_vars=None, metadata=meta)


def test_validators_and_mutators():
    v = CompositeValidator.default_config().set(validators=[
        ResourceLimitValidator.default_config().set(max_resources={"b200": 64}, denied_command_regex=r"rm -rf /")
    ]).instantiate()
    v.validate(_job({"b200": 64}))
    with pytest.raises(ValidationError, match="exceeds"):
        v.validate(_job({"b200": 128}))
    with pytest.raises(ValidationError, match="unknown resource"):
        v.validate(_job({"tpu": 1}))
    with pytest.raises(ValidationError, match="deny"):
        v.validate(_job({"b200": 8}, command="rm -rf / && python train.py"))
    pod = {"spec": {"tolerations": [{"key": "a"}], "containers": [{"name": "main"}], "hostNetwork": False}}
    patch = {"spec": {"tolerations": [{"key": "b"}], "hostNetwork": True, "priorityClassName": "high"}}
    out = MergePodMutator.default_config().set(patch=patch).instantiate().mutate(None, pod)
    assert out["spec"]["tolerations"] == [{"key": "a"}, {"key": "b"}] and out["spec"]["hostNetwork"] is True
    assert out["spec"]["priorityClassName"] == "high" and pod["spec"]["hostNetwork"] is False   # input untouched
    p = PrefixCommandPatcher.default_config().set(prefix="python -m axlearn_b200.ft.agent --").instantiate()
    assert p.patch("python train.py") == "python -m axlearn_b200.ft.agent -- python train.py"


def test_gcs_storage_helpers():
    from axlearn_b200.cloud.gcp import storage

    assert storage.split_url("gs://b/x/y") == ("b", "x/y")
    with pytest.raises(ValueError):
        storage.split_url("/local/path")
    listing = "gs://b/run/:\ngs://b/run/a.txt\ngs://b/run/sub/\ngs://b/run/sub/c.bin\n"
    rec = Recorder(outputs=[listing])
    assert storage.list_blobs("gs://b/run", runner=rec) == ["gs://b/run/a.txt", "gs://b/run/sub/c.bin"]
    assert rec.calls[0] == ["gcloud", "storage", "ls", "gs://b/run/**"]

    def missing(args, **kwargs):
        return types.SimpleNamespace(stdout="", stderr="matched no objects", returncode=1)

    assert storage.list_blobs("gs://b/none", runner=missing) == [] and not storage.blob_exists("gs://b/x", runner=missing)
    assert storage.blob_exists("gs://b/x", runner=Recorder(outputs=["gs://b/x\n"]))
    rec = Recorder()
    storage.upload_blob("/tmp/f", "gs://b/f", runner=rec)
    storage.download_blob("gs://b/f", "/tmp/g", runner=rec)
    storage.delete_blob("gs://b/dir", recursive=True, runner=rec)
    storage.sync_directory("/tmp/out", "gs://b/out", delete_unmatched=True, runner=rec)
    assert rec.calls == [["gcloud", "storage", "cp", "/tmp/f", "gs://b/f"],
                         ["gcloud", "storage", "cp", "gs://b/f", "/tmp/g"],
                         ["gcloud", "storage", "rm", "--recursive", "gs://b/dir"],
                         ["gcloud", "storage", "rsync", "--recursive", "--delete-unmatched-destination-objects",
                          "/tmp/out", "gs://b/out"]]
    with pytest.raises(RuntimeError, match="upload"):
        storage.upload_blob("/tmp/f", "gs://b/f", runner=missing)
