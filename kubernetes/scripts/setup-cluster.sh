#!/usr/bin/env bash
# Install what the chart needs on a fresh cluster: Kubeflow Trainer v2 (controller + its stock training runtimes)
# and Kueue.  Versions can be overridden from the environment.
set -euo pipefail
TRAINER_VERSION="${TRAINER_VERSION:-2.1.0}"
helm upgrade --install kubeflow-trainer oci://ghcr.io/kubeflow/charts/kubeflow-trainer \
  --namespace kubeflow-system --create-namespace --version "${TRAINER_VERSION}" \
  --set runtimes.defaultEnabled=true --wait --timeout 10m
kubectl apply --server-side -k "https://github.com/kubeflow/trainer.git/manifests/overlays/runtimes?ref=v${TRAINER_VERSION}"
kubectl -n kubeflow-system rollout status deploy/kubeflow-trainer-controller-manager --timeout=300s

KUEUE_VERSION="${KUEUE_VERSION:-v0.13.4}"
kubectl apply --server-side -f "https://github.com/kubernetes-sigs/kueue/releases/download/${KUEUE_VERSION}/manifests.yaml"
kubectl -n kueue-system rollout status deploy/kueue-controller-manager --timeout=300s
