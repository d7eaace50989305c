# Image for B200 machines (the reference's image, nvcr.io/nvidia/pytorch:23.06-py3, predates Blackwell).
# Needs a base with CUDA >= 12.8 (sm_100a support in nvcc) and PyTorch built for sm_100.
ARG BASE=nvcr.io/nvidia/pytorch:25.03-py3
FROM ${BASE}
WORKDIR /opt/stellatrain_b200
COPY . .
RUN python -m pip install --no-cache-dir pybind11 scipy pandas && python __graft_entry__.py
ENV PYTHONPATH=/opt/stellatrain_b200
CMD ["python", "-m", "stellatrain_b200"]
