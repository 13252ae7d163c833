# Container recipe for jaxpp_b200 (reference: scripts/docker/Dockerfile.base -- CUDA base image + Python environment).
# Needs a CUDA 12.8+ toolkit (nvcc with sm_100a), PyTorch 2.7+ built for CUDA 12.8 and the NCCL that ships with it.
#
#   docker build -t jaxpp_b200 .
#   docker run --gpus all --ipc=host --rm jaxpp_b200 tests/run_tests.sh
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv git \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
RUN pip install --no-cache-dir torch --index-url https://download.pytorch.org/whl/cu128 \
    && pip install --no-cache-dir numpy pytest pytest-timeout

WORKDIR /workspace/jaxpp_b200
COPY . .
# the native library has a C ABI and is built with plain nvcc for sm_100a (no GPU needed at build time)
RUN python -m jaxpp_b200.csrc.build
ENV PYTHONPATH=/workspace/jaxpp_b200 MASTER_ADDR=127.0.0.1
CMD ["python", "-m", "pytest", "tests", "-q", "-m", "not gpu"]
