"""Execution attestation records: which model, tokenizer, kernels and device produced an output.

A record fixes the backend, the device ordinal and architecture, SHA-256 digests of the canonical capability and
topology profiles, the numeric mode, the reproducibility class, the semantic versions of the kernels and of the
sampler, and the SHA-256 of the model and tokenizer files; ``attestation_sha256`` is the digest of the canonical JSON
of those fields, so a record is self-checking. Builders for the training/prefill route and for the decode runtime fix
the facts that are invariant for them (CUDA, bf16 storage with fp32 accumulation, numerical-equivalence
reproducibility across devices and bitwise repeatability on one device).

Counterparts in the reference: scirust-sciagent/src/execution_attestation.rs:16-61 (inputs and builder),
route_b_execution_attestation.rs:26-50 and cuda_decode_execution_attestation.rs (fixed facts of the two CUDA routes).
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass

SCHEMA_VERSION = 1
# Bumped whenever a kernel change alters results bit for bit (summation order, rounding point, tie rule).
KERNEL_SEMANTIC_VERSION = "scirust_b200.kernels/2"
SAMPLER_SEMANTIC_VERSION = "scirust_b200.sampler/1"      # fixed-point weights, radix select, xorshift64 streams
DECODE_SEMANTIC_VERSION = "scirust_b200.decode/2"        # fixed-order split-K GEMV, paged split-KV merge order


def sha256_hex(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def file_sha256(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


@dataclass
class ExecutionProfile:
    schema_version: int
    backend: str
    device_ordinal: int
    architecture_family: str
    architecture_name: str | None
    capability_profile_sha256: str
    topology_profile_sha256: str
    memory_budget_bytes: int | None
    numeric_mode: str
    reproducibility: str
    kernel_semantic_version: str
    sampler_semantic_version: str | None
    model_sha256: str
    tokenizer_sha256: str

    def canonical(self) -> bytes:
        return json.dumps(asdict(self), sort_keys=True, separators=(",", ":")).encode()


@dataclass
class ExecutionAttestation:
    profile: ExecutionProfile
    attestation_sha256: str

    @staticmethod
    def new(profile: ExecutionProfile) -> "ExecutionAttestation":
        for name in ("capability_profile_sha256", "topology_profile_sha256", "model_sha256", "tokenizer_sha256"):
            v = getattr(profile, name)
            if len(v) != 64 or any(c not in "0123456789abcdef" for c in v):
                raise ValueError(f"{name} must be 64 lowercase hex digits")
        if not profile.numeric_mode or not profile.kernel_semantic_version:
            raise ValueError("numeric_mode and kernel_semantic_version are required")
        return ExecutionAttestation(profile, sha256_hex(profile.canonical()))

    def verify(self) -> bool:
        return sha256_hex(self.profile.canonical()) == self.attestation_sha256

    def to_json(self) -> str:
        return json.dumps({"profile": asdict(self.profile), "attestation_sha256": self.attestation_sha256},
                          sort_keys=True, indent=2)

    @staticmethod
    def from_json(text: str) -> "ExecutionAttestation":
        d = json.loads(text)
        return ExecutionAttestation(ExecutionProfile(**d["profile"]), d["attestation_sha256"])


def device_profiles(device_index: int = 0):
    """Canonical capability / topology byte strings of a CUDA device (empty profiles without one)."""
    import torch
    if not torch.cuda.is_available():
        return b"capability:none", b"topology:none", None, None
    p = torch.cuda.get_device_properties(device_index)
    cap = (f"capability:v1;cc={p.major}.{p.minor};sms={p.multi_processor_count};"
           f"smem_optin={getattr(p, 'shared_memory_per_block_optin', 0)};l2={getattr(p, 'L2_cache_size', 0)}").encode()
    topo = f"topology:v1;devices={torch.cuda.device_count()};mem={p.total_memory}".encode()
    return cap, topo, p.total_memory, f"sm_{p.major}{p.minor}"


def build_training_route_attestation(model_sha256: str, tokenizer_sha256: str, device_index: int = 0,
                                     sampler: bool = False) -> ExecutionAttestation:
    """The resident bf16 training / prefill route on one CUDA device."""
    cap, topo, mem, arch = device_profiles(device_index)
    return ExecutionAttestation.new(ExecutionProfile(
        SCHEMA_VERSION, "cuda", device_index, "nvidia_gpu", arch, sha256_hex(cap), sha256_hex(topo), mem,
        "bf16 storage, fp32 accumulation", "numerical_equivalence_across_devices;bitwise_on_one_device",
        KERNEL_SEMANTIC_VERSION, SAMPLER_SEMANTIC_VERSION if sampler else None, model_sha256, tokenizer_sha256))


def build_decode_route_attestation(model_sha256: str, tokenizer_sha256: str, device_index: int = 0,
                                   weights: str = "bf16") -> ExecutionAttestation:
    """The cached decode runtime (paged KV, weight-streaming GEMV, device-side greedy feedback or sampler)."""
    cap, topo, mem, arch = device_profiles(device_index)
    return ExecutionAttestation.new(ExecutionProfile(
        SCHEMA_VERSION, "cuda", device_index, "nvidia_gpu", arch, sha256_hex(cap), sha256_hex(topo), mem,
        f"{weights} weights, bf16 activations and KV cache, fp32 accumulation",
        "numerical_equivalence_across_devices;bitwise_on_one_device", DECODE_SEMANTIC_VERSION,
        SAMPLER_SEMANTIC_VERSION, model_sha256, tokenizer_sha256))
