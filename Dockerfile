# Build and test image for flagcx-b200 (sm_100a only; nvcc cross-compiles without a GPU).
#
#   docker build -t flagcx-b200 .
#   docker run --gpus all --ipc=host --rm flagcx-b200 python -m pytest tests -q -m gpu
#
# The base image brings CUDA 12.9 (nvcc, cudart); PyTorch comes from its cu128 wheels,
# which bundle NCCL (the comparison arm of the benchmarks).
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04

RUN apt-get update && apt-get install -y --no-install-recommends \
        python3 python3-pip python3-dev python3-venv g++ make ninja-build git && \
    rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH CUDA_HOME=/usr/local/cuda
RUN pip install --no-cache-dir torch --index-url https://download.pytorch.org/whl/cu128 && \
    pip install --no-cache-dir numpy pytest pytest-timeout pybind11 ninja

WORKDIR /opt/flagcx-b200
COPY . .
# libflagcx.so, the torch backend, the fused-op extension, the bounds-checking build
RUN python -c "import __graft_entry__ as g; g.build()" && \
    make -C csrc install PREFIX=/usr/local && ldconfig && \
    pip install --no-cache-dir --no-build-isolation -e .
# CPU tier (sockets, shared-memory rings, bootstrap, host-side failure detection)
RUN python -m pytest tests -x -q -m "not gpu"
CMD ["python", "bench.py", "--help"]
