#!/usr/bin/env bash
# Install the controllers the chart needs: Kubeflow Trainer v2 and Kueue.
set -euo pipefail
TRAINER_VERSION="${TRAINER_VERSION:-v2.1.0}"
KUEUE_VERSION="${KUEUE_VERSION:-v0.13.4}"
kubectl apply --server-side -k "https://github.com/kubeflow/trainer.git/manifests/overlays/manager?ref=${TRAINER_VERSION}"
kubectl apply --server-side -f "https://github.com/kubernetes-sigs/kueue/releases/download/${KUEUE_VERSION}/manifests.yaml"
kubectl -n kubeflow-system rollout status deploy/kubeflow-trainer-controller-manager --timeout=300s
