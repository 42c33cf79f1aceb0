#!/usr/bin/env bash
# Log docker and the cluster into a container registry.  REGISTRY, REGISTRY_USER and REGISTRY_TOKEN come from the
# environment; nothing is stored in the repository.
set -euo pipefail
: "${REGISTRY:?set REGISTRY}" "${REGISTRY_USER:?set REGISTRY_USER}" "${REGISTRY_TOKEN:?set REGISTRY_TOKEN}"
echo "${REGISTRY_TOKEN}" | docker login "${REGISTRY}" --username "${REGISTRY_USER}" --password-stdin
kubectl create secret docker-registry b200moe-registry --docker-server="${REGISTRY}" \
  --docker-username="${REGISTRY_USER}" --docker-password="${REGISTRY_TOKEN}" --dry-run=client -o yaml | kubectl apply -f -
