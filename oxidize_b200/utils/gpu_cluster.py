"""GPU cluster profiles and Kubernetes manifest generator (``oxidize gpu-cluster``).

Covers the reference's ``cluster/gpu_cluster.rs`` (tier profiles for B200 / A100 / RTX Pro 6000
``:25-174``, node-pool / device-plugin / PrometheusRule emitters ``:232-436``, ``nvidia-smi`` CSV
parse + classify ``:458-514``).  Text generation only: nothing here changes a GPU setting.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional


@dataclass(frozen=True)
class GpuProfile:
    family: str
    display: str
    memory_gb: int
    gpus_per_node: int
    nvlink: bool
    instance_hint: str
    power_w: int


PROFILES: Dict[str, GpuProfile] = {
    "b200": GpuProfile("b200", "NVIDIA B200", 180, 8, True, "hgx-b200-8gpu", 1000),
    "a100": GpuProfile("a100", "NVIDIA A100 80GB", 80, 8, True, "a2-ultragpu-8g", 400),
    "rtx-pro-6000": GpuProfile("rtx-pro-6000", "NVIDIA RTX PRO 6000 Blackwell", 96, 4, False, "workstation-4gpu", 600),
}


def classify_gpu(name: str) -> Optional[str]:
    n = name.lower()
    if "b200" in n:
        return "b200"
    if "a100" in n:
        return "a100"
    if "rtx pro 6000" in n or "rtx 6000" in n:
        return "rtx-pro-6000"
    return None


def classify_inventory(names: List[str]) -> Dict[str, int]:
    out: Dict[str, int] = {}
    for n in names:
        k = classify_gpu(n) or "unknown"
        out[k] = out.get(k, 0) + 1
    return out


def render_cluster_manifests(cluster: str, family: str, nodes: int, image: str = "oxidize-b200:latest",
                             model_path: str = "/models/model.gguf") -> str:
    key = family.lower()
    if key not in PROFILES:
        raise ValueError(f"unknown GPU family {family!r}; have {sorted(PROFILES)}")
    p = PROFILES[key]
    tp = p.gpus_per_node if p.nvlink else 1
    docs = []
    docs.append(f"""apiVersion: v1
kind: Namespace
metadata:
  name: {cluster}
""")
    docs.append(f"""apiVersion: apps/v1
kind: DaemonSet
metadata:
  name: nvidia-device-plugin
  namespace: kube-system
spec:
  selector:
    matchLabels: {{name: nvidia-device-plugin}}
  template:
    metadata:
      labels: {{name: nvidia-device-plugin}}
    spec:
      tolerations:
        - {{key: nvidia.com/gpu, operator: Exists, effect: NoSchedule}}
      containers:
        - name: nvidia-device-plugin
          image: nvcr.io/nvidia/k8s-device-plugin:v0.17.0
          securityContext: {{allowPrivilegeEscalation: false}}
""")
    docs.append(f"""apiVersion: apps/v1
kind: Deployment
metadata:
  name: {cluster}-server
  namespace: {cluster}
  labels: {{app: {cluster}, gpu-family: {p.family}}}
spec:
  replicas: {nodes}
  selector:
    matchLabels: {{app: {cluster}}}
  template:
    metadata:
      labels: {{app: {cluster}}}
      annotations: {{prometheus.io/scrape: "true", prometheus.io/path: /metrics, prometheus.io/port: "8080"}}
    spec:
      nodeSelector: {{node.kubernetes.io/instance-type: {p.instance_hint}}}
      tolerations:
        - {{key: nvidia.com/gpu, operator: Exists, effect: NoSchedule}}
      containers:
        - name: oxidize
          image: {image}
          args: ["serve", "{model_path}", "--host", "0.0.0.0", "--port", "8080", "--backend", "cuda", "--tp", "{tp}"]
          ports: [{{containerPort: 8080}}]
          resources:
            limits: {{nvidia.com/gpu: {p.gpus_per_node}}}
          readinessProbe: {{httpGet: {{path: /readyz, port: 8080}}, periodSeconds: 5}}
          livenessProbe: {{httpGet: {{path: /livez, port: 8080}}, periodSeconds: 10}}
          volumeMounts: [{{name: models, mountPath: /models, readOnly: true}}, {{name: shm, mountPath: /dev/shm}}]
      volumes:
        - name: models
          persistentVolumeClaim: {{claimName: {cluster}-models}}
        - name: shm
          emptyDir: {{medium: Memory}}
""")
    docs.append(f"""apiVersion: v1
kind: Service
metadata:
  name: {cluster}
  namespace: {cluster}
spec:
  selector: {{app: {cluster}}}
  ports: [{{port: 80, targetPort: 8080}}]
""")
    docs.append(f"""apiVersion: monitoring.coreos.com/v1
kind: PrometheusRule
metadata:
  name: {cluster}-gpu-rules
  namespace: {cluster}
spec:
  groups:
    - name: gpu
      rules:
        - alert: GpuTemperatureHigh
          expr: DCGM_FI_DEV_GPU_TEMP > 85
          for: 5m
        - alert: GpuFramebufferNearlyFull
          expr: DCGM_FI_DEV_FB_USED / (DCGM_FI_DEV_FB_USED + DCGM_FI_DEV_FB_FREE) > 0.95
          for: 5m
        - alert: NvlinkReplayErrors
          expr: increase(DCGM_FI_DEV_NVLINK_REPLAY_ERROR_COUNT_TOTAL[5m]) > 0
        - alert: OxidizeQueueDeep
          expr: oxidize_queue_depth > 64
          for: 2m
""")
    return "---\n".join(docs)
