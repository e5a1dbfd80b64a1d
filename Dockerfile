# slopllm_b200: OpenAI-compatible server for GLM-5-class NVFP4 checkpoints on 8 x B200.
#
# Stage 1 (builder): the CUDA devel toolchain compiles every kernel for sm_100a (nvcc) and the host C++ runtime
# (g++) in-tree through `python -m slopllm_b200.build_native`.
# Stage 2 (runtime): CUDA runtime libraries, Python with PyTorch, and the built tree only.
#
#   docker build -t slopllm-b200 .
#   docker run --gpus all --ipc host --network host -v $HF_HOME:/hf-cache slopllm-b200
#
# The kernels target Blackwell B200 only (tcgen05 / TMEM / TMA); there is no other code path.
ARG CUDA_VERSION=12.9.1
FROM nvidia/cuda:${CUDA_VERSION}-devel-ubuntu24.04 AS builder

ARG TORCH_VERSION=2.11.0
ARG TORCH_INDEX=https://download.pytorch.org/whl/cu128
ENV DEBIAN_FRONTEND=noninteractive
RUN apt-get update && apt-get install -y --no-install-recommends \
        ca-certificates g++ make python3 python3-venv python3-dev \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
RUN pip install --no-cache-dir "torch==${TORCH_VERSION}" --index-url "${TORCH_INDEX}" \
    && pip install --no-cache-dir numpy safetensors transformers sentencepiece pyyaml prometheus_client

WORKDIR /opt/slopllm_b200
COPY slopllm_b200 ./slopllm_b200
COPY __graft_entry__.py bench.py README.md ./
# nvcc cross-compiles sm_100a without a GPU; the shared objects land in slopllm_b200/_lib
RUN python -m slopllm_b200.build_native

FROM nvidia/cuda:${CUDA_VERSION}-runtime-ubuntu24.04 AS runtime
ENV DEBIAN_FRONTEND=noninteractive
RUN apt-get update && apt-get install -y --no-install-recommends ca-certificates python3 curl \
    && rm -rf /var/lib/apt/lists/*
COPY --from=builder /opt/venv /opt/venv
COPY --from=builder /opt/slopllm_b200 /opt/slopllm_b200
ENV PATH=/opt/venv/bin:$PATH \
    PYTHONPATH=/opt/slopllm_b200 \
    PYTHONUNBUFFERED=1 \
    HF_HOME=/hf-cache
WORKDIR /opt/slopllm_b200
EXPOSE 8000
# One process per GPU over NCCL / NVLink; rank 0 listens.  Override CMD (or use docker-compose.yml) for other layouts.
CMD ["python", "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=8", "--master-addr", "127.0.0.1", \
     "-m", "slopllm_b200.cli.serve", "--model", "/models/glm", "--mtp", "--cp", "--host", "0.0.0.0", "--port", "8000"]
