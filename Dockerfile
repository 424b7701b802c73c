# Build and run image for a B200 (sm_100a) machine.
#   docker build -t flodl-b200 .
#   docker run --gpus all --ipc=host --rm flodl-b200 python bench.py --gpus 1
#   docker run --gpus all --ipc=host --rm flodl-b200 torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 bench.py --gpus 8
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04
ENV DEBIAN_FRONTEND=noninteractive PIP_NO_CACHE_DIR=1 PATH=/venv/bin:$PATH
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-venv python3-dev ninja-build g++ zlib1g-dev git graphviz \
    && rm -rf /var/lib/apt/lists/* && python3 -m venv /venv \
    && pip install torch numpy pybind11 pyyaml pytest pytest-timeout transformers safetensors sentencepiece nvidia-ml-py
WORKDIR /opt/flodl_b200
COPY . .
# nvcc cross-compiles sm_100a during the image build: no GPU is needed here
RUN python -c "import __graft_entry__ as g; g.build()" && python -m pytest tests -x -q -m "not gpu" -k "runtime or checkpoint or graph"
CMD ["python", "-m", "flodl_b200.cli", "diagnose"]
