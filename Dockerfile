# Build image for pie_b200 (sm_100a kernels + C++ host module). Needs a CUDA >= 12.8 toolchain.
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-dev g++ git \
    && rm -rf /var/lib/apt/lists/*
RUN pip3 install --break-system-packages torch numpy msgpack websockets safetensors regex pybind11 pillow scipy pytest
WORKDIR /opt/pie_b200
COPY . .
RUN python3 -m pie_b200._build
ENTRYPOINT ["python3", "-m", "pie_b200"]
CMD ["serve"]
