"""Where the worker processes of a run come from (tunix/experimental/distributed/deployment/*: local and k8s
contexts, JobSet YAML generator).

`LocalDeployment`  starts every worker as a child process of the controller on this host (`runtime.launcher`).
`jobset_manifest`  renders the same run as a Kubernetes JobSet: one replicated job per role, one pod per worker,
                   `nvidia.com/gpu` limits, the controller's directory address and the shared token handed to the
                   pods, each pod serving on its pod IP and running until it is terminated. The manifest is plain
                   data (`dict`); `to_yaml` writes it. Nothing here talks to a cluster: applying the manifest is
                   `kubectl apply -f`, outside this framework.

Both take the same `RoleSpec`s, so a run that works locally is deployed by changing the context, not the program."""
from __future__ import annotations

import dataclasses
import re
from typing import Optional, Sequence

from .launcher import Launcher


@dataclasses.dataclass
class RoleSpec:
    role: str                                               # "rollout", "trainer", ...
    factory: str                                            # "pkg.module:make_worker"
    replicas: int = 1
    gpus_per_worker: int = 0
    args: dict = dataclasses.field(default_factory=dict)
    port: int = 50051
    env: dict = dataclasses.field(default_factory=dict)

    def worker_ids(self) -> list:
        return [f"{self.role}-{i}" for i in range(self.replicas)]


class LocalDeployment:
    def __init__(self, roles: Sequence[RoleSpec], token: Optional[str] = None):
        self.roles, self.launcher = list(roles), Launcher(token)

    def start(self, timeout: float = 60.0) -> dict:
        ids = []
        for spec in self.roles:
            for wid in spec.worker_ids():
                self.launcher.launch(spec.factory, wid, role=spec.role, **spec.args)
                ids.append(wid)
        self.launcher.wait_for(ids, timeout)
        return self.launcher.workers()

    def shutdown(self, timeout: float = 10.0) -> None:
        self.launcher.shutdown(timeout)


_DNS = re.compile(r"^[a-z0-9]([-a-z0-9]*[a-z0-9])?$")


def _dns_name(s: str, what: str) -> str:
    if not _DNS.match(s) or len(s) > 63:
        raise ValueError(f"{what} {s!r} is not a DNS label (lower-case letters, digits and '-', at most 63 characters)")
    return s


def jobset_manifest(name: str, image: str, roles: Sequence[RoleSpec], *, directory_address: str,
                    token_secret: Optional[str] = None, namespace: str = "default", node_selector: Optional[dict] = None,
                    shm_size: str = "64Gi", python: str = "python") -> dict:
    """`directory_address` is where the controller's directory is reachable from the pods (a service name and port).
    `token_secret` names a Secret whose key `token` holds the shared call token."""
    _dns_name(name, "jobset name")
    jobs = []
    for spec in roles:
        _dns_name(spec.role, "role")
        if spec.replicas < 1:
            raise ValueError(f"role {spec.role!r}: replicas must be at least 1")
        cmd = [python, "-m", "tunix_b200.experimental.runtime.launcher", "--factory", spec.factory,
               "--worker-id", f"{spec.role}-$(JOB_COMPLETION_INDEX)", "--directory", directory_address,
               "--bind", f"0.0.0.0:{spec.port}", "--advertise", f"$(POD_IP):{spec.port}", "--stay",
               "--arg", f"role={spec.role}"]
        for k, v in spec.args.items():
            cmd += ["--arg", f"{k}={v}"]
        env = [{"name": "POD_IP", "valueFrom": {"fieldRef": {"fieldPath": "status.podIP"}}},
               {"name": "NCCL_DEBUG", "value": "WARN"}]
        env += [{"name": k, "value": str(v)} for k, v in spec.env.items()]
        if token_secret:
            env.append({"name": "TUNIX_B200_TOKEN", "valueFrom": {"secretKeyRef": {"name": token_secret, "key": "token"}}})
            cmd += ["--token", "$(TUNIX_B200_TOKEN)"]
        container = {"name": spec.role, "image": image, "command": cmd, "env": env,
                     "ports": [{"containerPort": spec.port, "name": "worker"}],
                     "volumeMounts": [{"name": "dshm", "mountPath": "/dev/shm"}]}
        if spec.gpus_per_worker:
            container["resources"] = {"limits": {"nvidia.com/gpu": spec.gpus_per_worker}}
        pod = {"restartPolicy": "Never", "containers": [container],
               "volumes": [{"name": "dshm", "emptyDir": {"medium": "Memory", "sizeLimit": shm_size}}]}   # NCCL wants a large /dev/shm
        if node_selector:
            pod["nodeSelector"] = dict(node_selector)
        jobs.append({"name": spec.role, "replicas": 1,
                     "template": {"spec": {"parallelism": spec.replicas, "completions": spec.replicas, "completionMode": "Indexed",
                                           "backoffLimit": 0, "template": {"metadata": {"labels": {"tunix-b200/role": spec.role}},
                                                                           "spec": pod}}}})
    return {"apiVersion": "jobset.x-k8s.io/v1alpha2", "kind": "JobSet",
            "metadata": {"name": name, "namespace": namespace},
            "spec": {"failurePolicy": {"maxRestarts": 0}, "replicatedJobs": jobs}}


def to_yaml(manifest: dict) -> str:
    import yaml
    return yaml.safe_dump(manifest, sort_keys=False, default_flow_style=False)
