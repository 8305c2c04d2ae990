# syntax=docker/dockerfile:1
# machx_inference_engine_b200: B200 (sm_100a) inference engine, build + runtime image.
#
#   docker build -t mx-b200 .
#   docker run --gpus all --ipc=host -p 11435:11435 -v /models:/models mx-b200 serve /models/gpt-oss-120b.gguf --gpus 8
#
# The build stage compiles the in-tree native libraries (g++ host library, nvcc kernels for sm_100a; no GPU is needed to build);
# the runtime stage carries the package, the built shared objects and PyTorch.  A host with B200 GPUs, driver 570+ and the NVIDIA
# container toolkit is required to run it; --ipc=host (or a large --shm-size) is needed for the one-process-per-GPU NCCL transport.

ARG BASE=nvcr.io/nvidia/pytorch:25.06-py3

# ============================ build stage ============================
FROM ${BASE} AS build
WORKDIR /src
COPY machx_inference_engine_b200 machx_inference_engine_b200
COPY __graft_entry__.py bench.py README.md ./
# nvcc -gencode arch=compute_100a,code=sm_100a for every kernel file; the result lands in machx_inference_engine_b200/_native/
RUN python -c "import __graft_entry__ as g; g.build()" \
 && ls -l machx_inference_engine_b200/_native/libmx_cuda.so machx_inference_engine_b200/_native/libmx_host.so

# ============================ runtime stage ============================
FROM ${BASE} AS runtime
ENV PYTHONUNBUFFERED=1 \
    NCCL_DEBUG=WARN
WORKDIR /opt/mx
COPY --from=build /src/machx_inference_engine_b200 machx_inference_engine_b200
COPY --from=build /src/bench.py /src/README.md ./
ENV PYTHONPATH=/opt/mx
EXPOSE 11435
# `serve --gpus N` re-launches itself with one rank per GPU; the server binds 0.0.0.0 inside the container.
ENTRYPOINT ["python", "-m", "machx_inference_engine_b200.cli.main"]
CMD ["--help"]
