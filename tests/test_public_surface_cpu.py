"""Every name a package lists in ``__all__`` resolves (lazy ones included), and the names a user of the reference imports
from the same places exist here."""

import importlib

import pytest

PACKAGES = ["phyai_b200", "phyai_b200.parallel", "phyai_b200.layers.linear", "phyai_b200.layers.attention", "phyai_b200.layers.layer_norm",
            "phyai_b200.layers.quant", "phyai_b200.layers.mlp", "phyai_b200.layers.vocab_embedding", "phyai_b200.layers.rotary_embedding",
            "phyai_b200.weights", "phyai_b200.cache", "phyai_b200.cache.radix_cache", "phyai_b200.runtime", "phyai_b200.vgpu", "phyai_b200.utils",
            "phyai_b200.tools", "phyai_b200.models.pi05", "phyai_b200.models.pi0", "phyai_b200.models.cosmos3"]


@pytest.mark.parametrize("name", PACKAGES)
def test_every_exported_name_resolves(name):
    mod = importlib.import_module(name)
    exported = list(getattr(mod, "__all__", [])) + list(getattr(mod, "_LAZY", []))
    assert exported, name
    missing = [n for n in exported if not hasattr(mod, n)]
    assert not missing, (name, missing)


# what code written against the reference imports, by package (library-specific backend classes left out)
EXPECTED = {
    "phyai_b200": ["Engine", "EngineArgs", "EngineConfig"],
    "phyai_b200.parallel": ["init", "all_reduce", "all_gather", "reduce_scatter", "all_to_all", "broadcast", "send", "recv", "barrier", "Mesh",
                            "Registry", "Dispatcher", "DefaultPolicy", "ForcedPolicy", "Policy", "NcclBackend", "GlooBackend", "TorchDistBackend",
                            "PyNCCLBackend", "get_dispatcher", "graph_capture", "CaptureUnsafeError", "NoBackendError"],
    "phyai_b200.layers.linear": ["ColumnParallelLinear", "RowParallelLinear", "QKVParallelLinear", "MergedColumnParallelLinear", "ReplicatedLinear",
                                 "KernelDispatcher", "LinearKernelRegistry", "register_linear_kernel", "list_registered_linear_kernels",
                                 "supported_specs_for_sm", "WeightSpec", "Bf16Spec", "Fp8Spec", "Nvfp4Spec", "AllocationRequest", "ActivationView"],
    "phyai_b200.layers.attention": ["Attention", "ARAttention", "DiffusionAttention", "AttnMetadata", "AttnCtx", "GatedDeltaNet", "GatedDeltaNetCtx",
                                    "list_attention_backends", "list_ar_backends", "list_diffusion_backends", "list_gdn_backends"],
    "phyai_b200.layers.quant": ["QuantScheme", "QuantPlan", "Matcher", "Rule", "load_quant_plan", "use_quant_plan", "get_active_plan", "materialize",
                                "WeightSpec", "LinearActivationQuant", "ActivationView"],
    "phyai_b200.weights": ["load_pretrained", "LoadReport", "WeightLoader", "sharded", "fused", "vocab", "replicated", "weight_norm_fold"],
    "phyai_b200.cache": ["KVCachePool", "StaticCache", "StaticCacheError", "CacheConfig", "PairedCache", "HybridCache", "MultimodalCache", "NestedCache"],
    "phyai_b200.runtime": ["ModelRunner", "Scheduler", "CudaGraph", "CudaGraphRegistry", "CudaGraphError", "CudaIpcBuffer", "HostShmBuffer", "TensorDumper",
                           "load_pass", "load_filter_fn", "register_tensor_dumper"],
    "phyai_b200.vgpu": ["init", "vGPU", "create_vgpus", "split_device", "split_device_by_sm_count", "register_vgpu_backend", "known_backends", "get_backend",
                        "set_backend", "GreenCtxBackend", "BackendCapabilityError"],
    "phyai_b200.utils": ["resolve_checkpoint", "find_safetensors", "load_config", "sm_arch", "init_cuda", "print_topology", "ProfilerConfig", "Profiler",
                         "NoOpProfiler", "TorchProfiler", "NsysProfiler", "make_profiler", "install_profiler", "set_profiler", "get_profiler", "event_scope",
                         "mark_instant", "add_profile_cli_args", "profile_config_from_args"],
    "phyai_b200.tools": ["BaseModelProcessor", "ProcessorPipeline", "ProcessorStep", "ProcessorStepRegistry", "__version__"],
    "phyai_b200.models.pi05": ["PI05Config", "PI05Model", "PI05VisionTower", "PaliGemmaLanguageModel", "PI05ExpertStack", "ActionTimeHeads", "PI05Request"],
    "phyai_b200.models.pi0": ["PI0Config", "PI0Model", "PI0ExpertStack", "ActionTimeHeads", "PaliGemmaLanguageModel", "PI0VisionTower", "GemmaExpertConfig",
                              "PI0Request"],
    "phyai_b200.models.cosmos3": ["Cosmos3Config", "Cosmos3Transformer", "Cosmos3Condition", "Cosmos3WanVAE", "Cosmos3AVAESoundDecoder",
                                  "Cosmos3T2VScheduler", "Cosmos3PolicyScheduler", "Cosmos3T2VWNScheduler", "Cosmos3PolicyWNScheduler", "Cosmos3T2VRunner",
                                  "Cosmos3ActionRunner", "UniPCMultistepSampler", "cosmos3_weight_remap", "cosmos3_vae_weight_remap",
                                  "cosmos3_avae_weight_remap"],
}


@pytest.mark.parametrize("name", sorted(EXPECTED))
def test_names_imported_from_the_reference_packages_exist(name):
    mod = importlib.import_module(name)
    missing = [n for n in EXPECTED[name] if not hasattr(mod, n)]
    assert not missing, (name, missing)


def test_profiler_factory_and_install():
    from phyai_b200.utils import NoOpProfiler, NsysProfiler, ProfilerConfig, get_profiler, install_profiler, make_profiler, set_profiler

    assert isinstance(make_profiler(None), NoOpProfiler) and isinstance(make_profiler(ProfilerConfig(kind="none")), NoOpProfiler)
    with pytest.raises(ValueError, match="unknown profiler kind"):
        make_profiler(ProfilerConfig(kind="perfetto"))
    mine = NoOpProfiler()
    assert set_profiler(mine) is mine and get_profiler() is mine
    assert isinstance(set_profiler(None), NoOpProfiler) and get_profiler() is not mine
    assert type(install_profiler(ProfilerConfig(kind="nsys"))) is NsysProfiler          # Nsight Systems reads the NVTX ranges
    install_profiler(None)
