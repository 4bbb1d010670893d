# Training image for 8x B200 (sm_100a) boxes: CUDA 12.9 toolchain for the in-tree kernel build, PyTorch with NCCL.
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04
ENV DEBIAN_FRONTEND=noninteractive PIP_NO_CACHE_DIR=1
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv g++ git numactl \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
RUN pip install torch --index-url https://download.pytorch.org/whl/cu128 \
    && pip install numpy safetensors pyyaml transformers pytest pytest-timeout pyarrow
WORKDIR /workspace/halo_b200
COPY . .
# nvcc cross-compiles for sm_100a without a GPU; the library lands in halo_b200/lib/
RUN python -c "import __graft_entry__ as g; g.build()"
# one process per GPU; CUDA_DEVICE_MAX_CONNECTIONS=1 keeps kernel launch order and collective order aligned
ENV CUDA_DEVICE_MAX_CONNECTIONS=1 NCCL_DEBUG=WARN
ENTRYPOINT ["python", "-m", "halo_b200.cli"]
