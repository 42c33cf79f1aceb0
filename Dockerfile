ARG BASE_IMAGE=b200moe-base:latest
FROM ${BASE_IMAGE}
WORKDIR /workspace/b200moe
COPY . .
# builds b200moe/_C/libb200moe.so for compute_100a/sm_100a (no GPU needed at build time)
RUN python -m b200moe.build
ENV PYTHONPATH=/workspace/b200moe
ENTRYPOINT ["torchrun", "--module", "distributed_parallel_training_pipelined"]
CMD ["--config-path", "configs/run_config.yaml"]
