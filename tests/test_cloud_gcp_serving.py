"""Serving-deployment manifests (LeaderWorkerSet, Service, probes, HPA, route, GKE policies)."""

import pytest

from axlearn_b200.cloud.common.pod_mutator import MergePodMutator
from axlearn_b200.cloud.gcp import serving


def _lws(**kw):
    return serving.LeaderWorkerSet.default_config().set(
        name="fuji-70b", image="reg/serve:v1", command="python -m axlearn_b200.inference.bench_decode --model 70B", **kw)


def test_leader_worker_set_pods():
    cfg = _lws(replicas=2, hosts_per_replica=2, env_vars={"NCCL_DEBUG": "WARN"}, service_account="sa",
               probes=[serving.StartupProbe.default_config(), serving.ReadinessProbe.default_config().set(path="/ready"),
                       serving.LivenessProbe.default_config().set(path=None)],
               pod_mutators=[MergePodMutator.default_config().set(patch={"spec": {"priorityClassName": "serving"}})])
    m = cfg.instantiate().build()
    assert m["apiVersion"] == serving.LWS_API and m["kind"] == "LeaderWorkerSet"
    spec = m["spec"]
    assert spec["replicas"] == 2 and spec["leaderWorkerTemplate"]["size"] == 2
    leader = spec["leaderWorkerTemplate"]["leaderTemplate"]
    worker = spec["leaderWorkerTemplate"]["workerTemplate"]
    lc, wc = leader["spec"]["containers"][0], worker["spec"]["containers"][0]
    assert lc["resources"]["limits"][serving.GPU_RESOURCE] == 8 == wc["resources"]["limits"][serving.GPU_RESOURCE]
    assert lc["ports"] == [{"containerPort": 8000, "name": "http"}] and "ports" not in wc
    assert lc["startupProbe"]["failureThreshold"] == 120 and lc["readinessProbe"]["httpGet"]["path"] == "/ready"
    assert lc["livenessProbe"]["tcpSocket"] == {"port": 8000} and "readinessProbe" not in wc
    env = {e["name"]: e["value"] for e in wc["env"]}
    assert env["MASTER_ADDR"] == "$(LWS_LEADER_ADDRESS)" and env["NODE_RANK"] == "$(LWS_WORKER_INDEX)"
    assert env["NCCL_DEBUG"] == "WARN" and env["NPROC_PER_NODE"] == "8"
    assert leader["spec"]["serviceAccountName"] == "sa" and leader["spec"]["priorityClassName"] == "serving"
    assert leader["spec"]["hostNetwork"] is True and leader["metadata"]["labels"]["role"] == "leader"
    assert _lws().instantiate().build()["spec"]["leaderWorkerTemplate"]["leaderTemplate"]["spec"]["hostNetwork"] is False
    with pytest.raises(ValueError):
        _lws(replicas=0).instantiate().build()
    with pytest.raises(ValueError):
        serving.ReadinessProbe.default_config().set(period_seconds=0).instantiate().build()


def test_service_hpa_route_and_policies():
    svc = serving.LWSService.default_config().set(name="m", ports=(80, 9090), target_ports=(8000, 9090),
                                                  port_names=("http", "metrics")).instantiate().build()
    assert svc["metadata"]["name"] == "m-service" and svc["spec"]["selector"]["role"] == "leader"
    assert svc["spec"]["ports"][1] == {"name": "metrics", "port": 9090, "targetPort": 9090, "protocol": "TCP"}
    with pytest.raises(ValueError):
        serving.LWSService.default_config().set(name="m", ports=(80,), target_ports=(1, 2)).instantiate().build()
    with pytest.raises(ValueError):
        serving.LWSService.default_config().set(name="m", service_type="Weird").instantiate().build()
    hpa = serving.HPA.default_config().set(
        name="m", min_replicas=1, max_replicas=8,
        metrics=[serving.HPAMetric.default_config().set(metric_name="requests_in_flight", average_value="16")])
    h = hpa.instantiate().build()
    assert h["spec"]["scaleTargetRef"] == {"apiVersion": serving.LWS_API, "kind": "LeaderWorkerSet", "name": "m"}
    assert h["spec"]["metrics"][0]["pods"]["target"] == {"type": "AverageValue", "averageValue": "16"}
    with pytest.raises(ValueError):
        hpa.clone(min_replicas=9).instantiate().build()
    with pytest.raises(ValueError):
        hpa.clone(metrics=[]).instantiate().build()
    route = serving.LWSHTTPRoute.default_config().set(name="m", hostnames=("llm.example",)).instantiate().build()
    assert route["spec"]["rules"][0]["matches"][0]["path"]["value"] == "/m"
    assert route["spec"]["rules"][1]["matches"][0]["headers"][0] == {"type": "Exact", "name": "x-model", "value": "m"}
    assert route["spec"]["rules"][0]["backendRefs"] == [{"name": "m-service", "port": 80}]
    assert serving.health_check_policy("m")["spec"]["targetRef"]["name"] == "m-service"
    assert serving.backend_policy("m", timeout_seconds=900)["spec"]["default"]["timeoutSec"] == 900
    assert serving.pod_monitoring("m")["spec"]["selector"]["matchLabels"] == {"app": "m", "role": "leader"}


class _Api:
    def __init__(self):
        self.applied, self.deleted = [], []

    def apply(self, manifest):
        self.applied.append(manifest)
        out = dict(manifest)
        out["metadata"] = {**manifest["metadata"], "uid": f"uid-{len(self.applied)}"}
        return out

    def delete(self, kind, namespace, name):
        self.deleted.append((kind, namespace, name))


def test_deployment_applies_set_first_and_owns_the_rest():
    dep = serving.ServingDeployment.default_config().set(
        lws=_lws(namespace="serving", port=9000),
        route=serving.LWSHTTPRoute.default_config(),
        hpa=serving.HPA.default_config().set(
            metrics=[serving.HPAMetric.default_config().set(metric_name="q", average_value="4")]),
        gke_policies=True, monitoring=True).instantiate()
    api = _Api()
    objs = dep.apply(api)
    kinds = [m["kind"] for m in api.applied]
    assert kinds == ["LeaderWorkerSet", "Service", "HTTPRoute", "HealthCheckPolicy", "GCPBackendPolicy",
                     "PodMonitoring", "HorizontalPodAutoscaler"]
    assert len(objs) == 7
    for m in api.applied[1:]:
        ref = m["metadata"]["ownerReferences"][0]
        assert ref["kind"] == "LeaderWorkerSet" and ref["name"] == "fuji-70b" and ref["uid"] == "uid-1"
        assert m["metadata"]["namespace"] == "serving"
    assert api.applied[1]["spec"]["ports"][0]["targetPort"] == 9000       # the set's port is the default target
    assert api.applied[3]["spec"]["default"]["config"]["httpHealthCheck"]["port"] == 9000
    dep.delete(api)
    assert api.deleted == [("LeaderWorkerSet", "serving", "fuji-70b")]


def test_cli_serve_manifest(capsys):
    import yaml

    from axlearn_b200.cli.main import main

    rc = main(["gcp", "serve-manifest", "--name", "m7", "--image", "reg/serve:v1", "--num_nodes", "2", "--replicas", "1",
               "--max_replicas", "3", "--gateway", "gw", "--", "python", "-m", "server"])
    assert rc == 0
    objs = [o for o in yaml.safe_load_all(capsys.readouterr().out) if o]
    assert [o["kind"] for o in objs] == ["LeaderWorkerSet", "Service", "HTTPRoute", "HealthCheckPolicy",
                                         "GCPBackendPolicy", "PodMonitoring", "HorizontalPodAutoscaler"]
    lws = objs[0]["spec"]["leaderWorkerTemplate"]
    assert lws["size"] == 2 and lws["leaderTemplate"]["spec"]["containers"][0]["command"][-1] == "python -m server"
    assert objs[-1]["spec"]["maxReplicas"] == 3 and objs[2]["spec"]["parentRefs"][0]["name"] == "gw"
