# Container recipe for crossbow_b200 (counterpart of the reference's tools/dockerfiles/dockerfiles/crossbow-cuda-9.2.Dockerfile,
# which pins CUDA 9.2 / cuDNN 7.1 / NCCL 2 / OpenBLAS / libjpeg-turbo).  This framework needs none of cuDNN, cuBLAS, OpenBLAS
# or libjpeg: its kernels and its JPEG decoder are its own.  It needs the CUDA 12.9 toolkit (nvcc with sm_100a), PyTorch with
# NCCL for the process group, and a Blackwell GPU at run time (driver >= 575).
#
#   docker build -t crossbow-b200 .
#   docker run --gpus all --ipc=host --rm crossbow-b200 python bench.py --gpus 1
#   docker run --gpus all --ipc=host --rm crossbow-b200 \
#       python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench.py --gpus 8
#
# (--ipc=host: the ranks exchange CUDA IPC handles of their peer buffers.)
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

ENV DEBIAN_FRONTEND=noninteractive PIP_BREAK_SYSTEM_PACKAGES=1 PYTHONUNBUFFERED=1
RUN apt-get update && apt-get install -y --no-install-recommends \
        python3 python3-pip python3-dev g++ make git && \
    rm -rf /var/lib/apt/lists/* && ln -sf /usr/bin/python3 /usr/bin/python

# PyTorch (tensor / process-group layer), NumPy, NVML bindings for the read-only clock sampler, Pillow + pytest for the tests
RUN pip install --no-cache-dir --index-url https://download.pytorch.org/whl/cu128 torch && \
    pip install --no-cache-dir numpy nvidia-ml-py pillow pytest

ENV CROSSBOW_HOME=/opt/crossbow_b200
WORKDIR ${CROSSBOW_HOME}
COPY . ${CROSSBOW_HOME}

# build libxbow_cuda.so (sm_100a kernels + device executor) and libxbow_rt.so (host runtime) in-tree; nvcc cross-compiles
# without a GPU, so this works in `docker build`
RUN python -c "import __graft_entry__ as g; g.build()"

# host-only tests (no GPU needed at build time)
RUN python -m pytest tests -q -x -m "not gpu" -p no:cacheprovider

CMD ["python", "bench.py", "--gpus", "1"]
