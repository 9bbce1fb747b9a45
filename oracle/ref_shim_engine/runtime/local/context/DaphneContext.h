// TEST INFRASTRUCTURE.  Stand-in for DAPHNE's DaphneContext when the reference's vectorized ENGINE (MTWrapper, tasks,
// workers) is compiled as the CPU baseline: the real header pulls in the compiler (MLIR) through DaphneUserConfig.h.
// It carries exactly the members the engine reads (vectorized/MTWrapper.h:153-211, MTWrapper_dense.cpp:24-200,
// kernels/VectorizedPipeline.h:53-57, vectorized/WorkerCPU.h): the user configuration with DAPHNE's defaults
// (api/cli/DaphneUserConfig.h), a logger, and an empty list of CUDA contexts.
#pragma once

#include <runtime/local/vectorized/LoadPartitioningDefs.h>

#include <spdlog/spdlog.h>

#include <memory>
#include <vector>

struct EngineUserConfig {
    bool vectorized_single_queue = false;
    bool prePartitionRows = false;
    bool pinWorkers = false;
    bool hyperthreadingEnabled = false;
    bool debugMultiThreading = false;
    bool use_cuda = false;
    SelfSchedulingScheme taskPartitioningScheme = SelfSchedulingScheme::STATIC;
    QueueTypeOption queueSetupScheme = QueueTypeOption::CENTRALIZED;
    VictimSelectionLogic victimSelection = VictimSelectionLogic::SEQPRI;
    int numberOfThreads = -1;
    int minimumTaskSize = 1;
    size_t phyBatchSize = 96 * 1024; // bytes of inputs + outputs per batch of a task
};

struct DaphneContext {
    EngineUserConfig config;
    std::vector<void *> cuda_contexts;
    std::shared_ptr<spdlog::logger> logger = std::make_shared<spdlog::logger>("runtime");
    EngineUserConfig &getUserConfig() { return config; }
    [[nodiscard]] bool useCUDA() const { return false; }
};
#define DCTX(varname) DaphneContext *varname
