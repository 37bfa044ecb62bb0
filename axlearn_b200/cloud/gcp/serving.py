"""Kubernetes objects for multi-host SERVING deployments on GKE: a LeaderWorkerSet of B200 pods
and what fronts it (reference: axlearn/cloud/gcp/lws_utils.py:21-159, k8s_service.py:36-245,
k8s_readiness_probe.py:13-277, k8s_hpa.py:28-250, k8s_http_route.py:133-341,
k8s_health_check_policy.py:19, k8s_backend_policy.py:19, k8s_metrics_collection.py:48-250).

A decode deployment of this framework is one process per GPU on one or more hosts
(``python -m axlearn_b200.inference...`` under torchrun); a LeaderWorkerSet replica is such a group
of hosts, the leader pod terminates HTTP, and replicas scale with load.  Every builder returns a
plain manifest dict; ``ServingDeployment`` bundles them and applies them through the same
``KubernetesApi``-style object the training jobs use (anything with ``apply(manifest)`` /
``delete(kind, namespace, name)``), so the tests run against a recorder.
"""

from __future__ import annotations

from typing import Any, Optional, Sequence

from axlearn_b200.common.config import REQUIRED, Configurable, Required, config_class

LWS_API = "leaderworkerset.x-k8s.io/v1"
GPU_RESOURCE = "nvidia.com/gpu"


def _meta(name: str, namespace: str, labels: Optional[dict] = None) -> dict:
    out = {"name": name, "namespace": namespace}
    if labels:
        out["labels"] = dict(labels)
    return out


def owner_reference(owner: dict) -> dict:
    """Ties an object's lifetime to ``owner`` (deleted with it by the garbage collector)."""
    return {"apiVersion": owner["apiVersion"], "kind": owner["kind"], "name": owner["metadata"]["name"],
            "uid": owner["metadata"].get("uid", ""), "controller": True, "blockOwnerDeletion": True}


class ContainerProbe(Configurable):
    """One of the three kubelet probes, as an HTTP GET or a TCP connect on a port."""

    KIND = "probe"

    @config_class
    class Config(Configurable.Config):
        port: int = 8000
        path: Optional[str] = "/healthz"       # None = TCP socket probe
        initial_delay_seconds: int = 0
        period_seconds: int = 10
        timeout_seconds: int = 5
        failure_threshold: int = 3
        success_threshold: int = 1

    def build(self) -> dict:
        cfg = self._config
        if cfg.period_seconds <= 0 or cfg.timeout_seconds <= 0 or cfg.failure_threshold <= 0:
            raise ValueError("period, timeout and failure threshold must be positive")
        action = ({"httpGet": {"path": cfg.path, "port": cfg.port}} if cfg.path is not None
                  else {"tcpSocket": {"port": cfg.port}})
        return {**action, "initialDelaySeconds": cfg.initial_delay_seconds, "periodSeconds": cfg.period_seconds,
                "timeoutSeconds": cfg.timeout_seconds, "failureThreshold": cfg.failure_threshold,
                "successThreshold": cfg.success_threshold}


class ReadinessProbe(ContainerProbe):
    KIND = "readinessProbe"


class LivenessProbe(ContainerProbe):
    KIND = "livenessProbe"

    @config_class
    class Config(ContainerProbe.Config):
        failure_threshold: int = 6


class StartupProbe(ContainerProbe):
    """Loading tens of GB of weights takes minutes: the other probes only start once this passes."""

    KIND = "startupProbe"

    @config_class
    class Config(ContainerProbe.Config):
        period_seconds: int = 15
        failure_threshold: int = 120


class LeaderWorkerSet(Configurable):
    """``replicas`` groups of ``hosts_per_replica`` pods with ``gpus_per_host`` B200s each; pod 0 of
    a group is the leader (HTTP front end and rank 0), the others are workers that join its
    rendezvous through the LWS-provided leader address."""

    @config_class
    class Config(Configurable.Config):
        name: Required[str] = REQUIRED
        namespace: str = "default"
        image: Required[str] = REQUIRED
        command: Required[str] = REQUIRED
        replicas: int = 1
        hosts_per_replica: int = 1
        gpus_per_host: int = 8
        machine_type: str = "a4-highgpu-8g"
        env_vars: dict = {}
        service_account: Optional[str] = None
        port: int = 8000
        probes: Sequence = ()
        restart_policy: str = "RecreateGroupOnPodRestart"
        pod_mutators: Sequence = ()

    def _pod_template(self, *, leader: bool) -> dict:
        cfg = self._config
        env = [{"name": k, "value": str(v)} for k, v in sorted(cfg.env_vars.items())]
        env += [
            # The LWS controller injects the leader's stable address and the group size.
            {"name": "MASTER_ADDR", "value": "$(LWS_LEADER_ADDRESS)"},
            {"name": "MASTER_PORT", "value": "29500"},
            {"name": "NNODES", "value": "$(LWS_GROUP_SIZE)"},
            {"name": "NODE_RANK", "value": "$(LWS_WORKER_INDEX)"},
            {"name": "NPROC_PER_NODE", "value": str(cfg.gpus_per_host)},
        ]
        container = {
            "name": "main", "image": cfg.image, "command": ["bash", "-c", cfg.command], "env": env,
            "resources": {"limits": {GPU_RESOURCE: cfg.gpus_per_host}},
            "volumeMounts": [{"name": "shm", "mountPath": "/dev/shm"}],
        }
        if leader:
            container["ports"] = [{"containerPort": cfg.port, "name": "http"}]
            for probe_cfg in cfg.probes:
                probe = probe_cfg.instantiate()
                container[probe.KIND] = probe.build()
        spec = {
            "containers": [container],
            "nodeSelector": {"node.kubernetes.io/instance-type": cfg.machine_type},
            "tolerations": [{"key": GPU_RESOURCE, "operator": "Exists", "effect": "NoSchedule"}],
            "volumes": [{"name": "shm", "emptyDir": {"medium": "Memory"}}],
            "hostNetwork": cfg.hosts_per_replica > 1, "dnsPolicy": "ClusterFirstWithHostNet",
        }
        if cfg.service_account:
            spec["serviceAccountName"] = cfg.service_account
        pod = {"metadata": {"labels": {"app": cfg.name, "role": "leader" if leader else "worker"}}, "spec": spec}
        for mutator_cfg in cfg.pod_mutators:
            pod = mutator_cfg.instantiate().mutate(None, pod)
        return pod

    def build(self) -> dict:
        cfg = self._config
        if cfg.replicas < 1 or cfg.hosts_per_replica < 1:
            raise ValueError("replicas and hosts_per_replica must be at least 1")
        template: dict[str, Any] = {"size": cfg.hosts_per_replica, "workerTemplate": self._pod_template(leader=False),
                                    "restartPolicy": cfg.restart_policy}
        template["leaderTemplate"] = self._pod_template(leader=True)
        return {"apiVersion": LWS_API, "kind": "LeaderWorkerSet", "metadata": _meta(cfg.name, cfg.namespace),
                "spec": {"replicas": cfg.replicas, "leaderWorkerTemplate": template,
                         "startupPolicy": "LeaderCreated"}}


class LWSService(Configurable):
    """A Service that selects the LEADER pods of a LeaderWorkerSet."""

    @config_class
    class Config(Configurable.Config):
        name: Required[str] = REQUIRED
        namespace: str = "default"
        service_type: str = "ClusterIP"
        ports: Sequence[int] = (80,)
        target_ports: Sequence[int] = (8000,)
        protocols: Sequence[str] = ("TCP",)
        port_names: Optional[Sequence[str]] = None

    def build(self, owner: Optional[dict] = None) -> dict:
        cfg = self._config
        if not (len(cfg.ports) == len(cfg.target_ports)):
            raise ValueError("ports and target_ports must have the same length")
        if cfg.service_type not in ("ClusterIP", "NodePort", "LoadBalancer"):
            raise ValueError(f"unknown service type {cfg.service_type!r}")
        ports = []
        for i, (port, target) in enumerate(zip(cfg.ports, cfg.target_ports)):
            proto = cfg.protocols[i] if i < len(cfg.protocols) else cfg.protocols[-1]
            name = cfg.port_names[i] if cfg.port_names else f"port-{port}"
            ports.append({"name": name, "port": int(port), "targetPort": int(target), "protocol": proto})
        meta = _meta(f"{cfg.name}-service", cfg.namespace)
        if owner is not None:
            meta["ownerReferences"] = [owner_reference(owner)]
        return {"apiVersion": "v1", "kind": "Service", "metadata": meta,
                "spec": {"type": cfg.service_type, "ports": ports,
                         "selector": {"leaderworkerset.sigs.k8s.io/name": cfg.name, "role": "leader"}}}


class HPAMetric(Configurable):
    """A per-pod custom metric (e.g. queue depth or tokens in flight exported by the server)."""

    @config_class
    class Config(Configurable.Config):
        metric_name: Required[str] = REQUIRED
        average_value: Required[str] = REQUIRED      # Kubernetes quantity, e.g. "8" or "500m"

    def build(self) -> dict:
        cfg = self._config
        return {"type": "Pods", "pods": {"metric": {"name": cfg.metric_name},
                                         "target": {"type": "AverageValue", "averageValue": str(cfg.average_value)}}}


class HPA(Configurable):
    """HorizontalPodAutoscaler (autoscaling/v2) over the LeaderWorkerSet's replicas."""

    @config_class
    class Config(Configurable.Config):
        name: Required[str] = REQUIRED
        namespace: str = "default"
        min_replicas: int = 1
        max_replicas: int = 4
        metrics: Sequence = ()
        scale_down_stabilization_seconds: int = 300

    def build(self, owner: Optional[dict] = None) -> dict:
        cfg = self._config
        if not 1 <= cfg.min_replicas <= cfg.max_replicas:
            raise ValueError("need 1 <= min_replicas <= max_replicas")
        if not cfg.metrics:
            raise ValueError("an HPA needs at least one metric")
        meta = _meta(f"{cfg.name}-hpa", cfg.namespace)
        if owner is not None:
            meta["ownerReferences"] = [owner_reference(owner)]
        return {"apiVersion": "autoscaling/v2", "kind": "HorizontalPodAutoscaler", "metadata": meta,
                "spec": {"scaleTargetRef": {"apiVersion": LWS_API, "kind": "LeaderWorkerSet", "name": cfg.name},
                         "minReplicas": cfg.min_replicas, "maxReplicas": cfg.max_replicas,
                         "metrics": [m.instantiate().build() for m in cfg.metrics],
                         "behavior": {"scaleDown": {"stabilizationWindowSeconds": cfg.scale_down_stabilization_seconds}}}}


class LWSHTTPRoute(Configurable):
    """Gateway-API HTTPRoute from a shared gateway to the leader Service: requests under
    ``/{name}/`` (or with the ``x-model`` header naming the deployment) go to it, prefix stripped."""

    @config_class
    class Config(Configurable.Config):
        name: Required[str] = REQUIRED
        namespace: str = "default"
        gateway_name: str = "inference-gateway"
        gateway_namespace: str = "default"
        service_port: int = 80
        hostnames: Sequence[str] = ()
        timeout_seconds: int = 600

    def build(self, owner: Optional[dict] = None) -> dict:
        cfg = self._config
        backend = [{"name": f"{cfg.name}-service", "port": cfg.service_port}]
        timeouts = {"request": f"{cfg.timeout_seconds}s", "backendRequest": f"{cfg.timeout_seconds}s"}
        rules = [
            {"matches": [{"path": {"type": "PathPrefix", "value": f"/{cfg.name}"}}],
             "filters": [{"type": "URLRewrite",
                          "urlRewrite": {"path": {"type": "ReplacePrefixMatch", "replacePrefixMatch": "/"}}}],
             "backendRefs": backend, "timeouts": timeouts},
            {"matches": [{"headers": [{"type": "Exact", "name": "x-model", "value": cfg.name}]}],
             "backendRefs": backend, "timeouts": timeouts},
        ]
        meta = _meta(f"{cfg.name}-route", cfg.namespace)
        if owner is not None:
            meta["ownerReferences"] = [owner_reference(owner)]
        spec: dict[str, Any] = {"parentRefs": [{"name": cfg.gateway_name, "namespace": cfg.gateway_namespace}],
                                "rules": rules}
        if cfg.hostnames:
            spec["hostnames"] = list(cfg.hostnames)
        return {"apiVersion": "gateway.networking.k8s.io/v1", "kind": "HTTPRoute", "metadata": meta, "spec": spec}


def health_check_policy(name: str, namespace: str = "default", *, port: int = 8000, path: str = "/healthz",
                        owner: Optional[dict] = None) -> dict:
    """GKE load-balancer health check for the leader Service (the default probes ``/`` on the
    serving port, which a model server does not answer)."""
    meta = _meta(f"{name}-health", namespace)
    if owner is not None:
        meta["ownerReferences"] = [owner_reference(owner)]
    return {"apiVersion": "networking.gke.io/v1", "kind": "HealthCheckPolicy", "metadata": meta,
            "spec": {"default": {"config": {"type": "HTTP", "httpHealthCheck": {"port": port, "requestPath": path}}},
                     "targetRef": {"group": "", "kind": "Service", "name": f"{name}-service"}}}


def backend_policy(name: str, namespace: str = "default", *, timeout_seconds: int = 600,
                   owner: Optional[dict] = None) -> dict:
    """GKE backend policy: long generation requests must outlive the load balancer's default 30 s."""
    meta = _meta(f"{name}-backend", namespace)
    if owner is not None:
        meta["ownerReferences"] = [owner_reference(owner)]
    return {"apiVersion": "networking.gke.io/v1", "kind": "GCPBackendPolicy", "metadata": meta,
            "spec": {"default": {"timeoutSec": timeout_seconds, "connectionDraining": {"drainingTimeoutSec": 60}},
                     "targetRef": {"group": "", "kind": "Service", "name": f"{name}-service"}}}


def pod_monitoring(name: str, namespace: str = "default", *, port: str = "http", path: str = "/metrics",
                   interval: str = "15s", owner: Optional[dict] = None) -> dict:
    """Managed-Prometheus scrape of the leaders' metrics endpoint (what the HPA's pod metrics read)."""
    meta = _meta(f"{name}-monitoring", namespace)
    if owner is not None:
        meta["ownerReferences"] = [owner_reference(owner)]
    return {"apiVersion": "monitoring.googleapis.com/v1", "kind": "PodMonitoring", "metadata": meta,
            "spec": {"selector": {"matchLabels": {"app": name, "role": "leader"}},
                     "endpoints": [{"port": port, "path": path, "interval": interval}]}}


class ServingDeployment(Configurable):
    """The LeaderWorkerSet plus its Service and, optionally, route, policies, monitoring and HPA.
    ``apply`` creates the set first and hands its (server-assigned) identity to the others as their
    owner, so deleting the set removes everything."""

    @config_class
    class Config(Configurable.Config):
        lws: Required[Any] = REQUIRED                 # LeaderWorkerSet.Config
        service: Optional[Any] = None                 # LWSService.Config (default: port 80 -> the set's port)
        route: Optional[Any] = None                   # LWSHTTPRoute.Config
        hpa: Optional[Any] = None                     # HPA.Config
        gke_policies: bool = False
        monitoring: bool = False

    def manifests(self, owner: Optional[dict] = None) -> list[dict]:
        cfg = self._config
        lws_cfg = cfg.lws
        name, ns = lws_cfg.name, lws_cfg.namespace
        service_cfg = cfg.service or LWSService.default_config().set(target_ports=(lws_cfg.port,))
        out = [service_cfg.clone(name=name, namespace=ns).instantiate().build(owner)]
        if cfg.route is not None:
            out.append(cfg.route.clone(name=name, namespace=ns).instantiate().build(owner))
        if cfg.gke_policies:
            out.append(health_check_policy(name, ns, port=lws_cfg.port, owner=owner))
            out.append(backend_policy(name, ns, owner=owner))
        if cfg.monitoring:
            out.append(pod_monitoring(name, ns, owner=owner))
        if cfg.hpa is not None:
            out.append(cfg.hpa.clone(name=name, namespace=ns).instantiate().build(owner))
        return out

    def apply(self, api: Any) -> list[dict]:
        created = api.apply(self._config.lws.instantiate().build())
        owner = created if isinstance(created, dict) and "metadata" in created else None
        rest = self.manifests(owner)
        for m in rest:
            api.apply(m)
        return [created] + rest

    def delete(self, api: Any) -> None:
        cfg = self._config.lws
        api.delete("LeaderWorkerSet", cfg.namespace, cfg.name)
