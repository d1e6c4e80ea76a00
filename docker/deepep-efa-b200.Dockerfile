# Container recipe for deepep_efa_b200 on one NVSwitch box of B200s.
#
# One stage: CUDA 12.9 toolkit (nvcc for sm_100a), PyTorch cu128/cu129 wheels, the package built in-tree for sm_100a at
# image build time (nvcc cross-compiles, no GPU needed). No libfabric, GDRCopy or EFA installer: inside one NVLink domain
# all traffic is peer loads and stores issued by the kernels.
# The reference's recipe (docker/deepep-efa.Dockerfile) additionally builds GDRCopy and the EFA user space.
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

RUN apt-get update && \
    apt-get install -y --no-install-recommends git build-essential ninja-build python3-dev python3-pip python3-venv && \
    apt-get clean && rm -rf /var/lib/apt/lists/*

ENV PIP_BREAK_SYSTEM_PACKAGES=1
RUN python3 -m pip install torch --index-url https://download.pytorch.org/whl/cu129 && \
    python3 -m pip install numpy ninja pytest pybind11 nvidia-ml-py

WORKDIR /app/deepep_efa_b200
COPY . .

# Build the extension for sm_100a into deepep_efa_b200/_build (the .so is found there at import; nothing is installed
# into site-packages) and run the CPU-only part of the test suite as a build check.
RUN python3 -c "import __graft_entry__ as g; g.build()" && \
    python3 -m pytest tests -q -m "not gpu"

ENV PYTHONPATH=/app/deepep_efa_b200
# 8 GPUs of one box: headline benchmark, then the GPU test suite
CMD ["bash", "launch.sh", "bench", "8"]
