#!/usr/bin/env bash
# Log docker into the Nebius container registries of the regions training images are pushed to.
# REGIONS overrides the list; the token comes from the `nebius` CLI of the logged-in user, nothing is stored here.
set -euo pipefail
REGIONS="${REGIONS:-us-central1 us-north1 uk-south1 eu-west2}"
for region in ${REGIONS}; do
  nebius iam get-access-token | docker login "cr.${region}.nebius.cloud" --username iam --password-stdin
done
