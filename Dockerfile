# Build and test image for torchft_b200.  nvcc cross-compiles the sm_100a kernel library, so the image builds
# on a machine without a GPU; the GPU tests and benchmarks need a B200 at run time (`docker run --gpus all`).
FROM nvidia/cuda:12.9.0-devel-ubuntu22.04

RUN apt-get update && apt-get install -y --no-install-recommends python3.12 python3.12-venv python3-pip g++ git \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m pip install --no-cache-dir torch numpy pybind11 pytest pytest-timeout psutil

WORKDIR /workspace/torchft_b200
COPY . .
RUN python3 -c "import __graft_entry__ as g; g.build()"

# CPU suite by default; on a B200: docker run --gpus all <image> python3 -m pytest tests -q -m gpu
CMD ["python3", "-m", "pytest", "tests", "-q", "-m", "not gpu"]
