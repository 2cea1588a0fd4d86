"""saber_engine_b200: a Blackwell-native (sm_100a) LLM inference engine with the capabilities of
GGZ14/saber-engine: `saber models` / `saber serve`, an OpenAI-compatible server, one resolved launch
plan, SBRPACK1 packs (W4A8-iu8 / MXFP4 / NVFP4), paged KV with prefix caching, block speculative
decoding, CUDA-graph decode buckets, the dense 27B hybrid and a Flash-Next-style MoE."""
__version__ = "0.1.0"
