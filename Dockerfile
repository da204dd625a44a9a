# CUDA 12.9 development image with PyTorch; the sm_100a kernels are compiled in-tree at build time
# (nvcc cross-compiles without a GPU) so the container starts with a ready library.
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv git && \
    rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
RUN pip install --no-cache-dir torch numpy pyyaml pytest
WORKDIR /workspace/ironcore_b200
COPY . .
RUN python -m ironcore_b200.ops.build
ENTRYPOINT ["python", "-m", "ironcore_b200"]
