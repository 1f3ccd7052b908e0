// Driver for the reference's single-GPU engine, written against its public API (the call sequence of its own
// tests/test_single_node_fullgpu_training.cc, whose dataset path, device index and model size are hard-coded).
// Nothing of the reference is modified: this file only parses four arguments, builds the GCN of applications/gcn.cc
// (per layer: weight, matmul, aggregation, then ReLU or softmax) and hands it to SingleNodeExecutionEngineGPU with
// OperatorExecutorGPUV2, AdamOptimizerGPU and CrossEntropyLossGPU.  The engine prints its own per-epoch lines and
// its "Average per-epoch runtime" (wall clock, first five epochs excluded), which the caller parses.
//
//   reference_gpu_driver DATASET_DIR LAYERS HIDDEN EPOCHS [ENGINE]
//     ENGINE  single (default) : SingleNodeExecutionEngineGPU, one process
//             hybrid           : DistributedPIPHybridParallelExecutionEngineGPU (tests/test_cuda_pipeline_parallel.cc);
//                                exactly 4 ranks, its built-in partition table, stage and halo traffic staged through
//                                host memory and MPI
//             model            : DistributedModelParallelExecutionEngineGPU (tests/test_cuda_model_parallel.cc); NCCL
//                                point-to-point between consecutive ranks, communicator bootstrapped over MPI as there
//     The multi-rank engines are started with baseline/shims/mpirun_local.py; Context::init_context binds rank r to GPU r.
//
// No train/validation/test masks are set: the reference's masked loss kernels index the per-vertex mask with
// vertex*classes+class (core/src/cuda/cuda_loss.cu:69-93), which reads past the end of the mask.
#include <assert.h>
#include <stdio.h>
#include <stdlib.h>

#include <string>

#include "application.h"
#include "context.h"
#include "engine.h"
#include "executor.h"
#include "graph.h"
#include "graph_loader.h"
#include "types.h"
#include "cuda/cuda_executor.h"
#include "cuda/cuda_graph.h"
#include "cuda/cuda_graph_loader.h"
#include "cuda/cuda_loss.h"
#include "cuda/cuda_optimizer.h"
#include "cuda/cuda_single_cpu_engine.h"
#include "cuda/cuda_hybrid_parallel.h"
#include "cuda/cuda_model_parallel.h"
#include "cuda/cuda_utils.h"
#include "distributed_sys.h"

class DriverGCN : public AbstractApplication {
    int layers_, hidden_, classes_;

  public:
    DriverGCN(int layers, int hidden, int classes, int features)
        : AbstractApplication(features), layers_(layers), hidden_(hidden), classes_(classes) {}
    Tensor* forward(Tensor* input) {
        Tensor* t = input;
        for (int i = 0; i < layers_; ++i) {
            const bool last = i == layers_ - 1;
            Tensor* w = weight(t->dims[1], last ? classes_ : hidden_);
            t = matmul(t, w);
            t = aggregation(t, NORM_SUM);
            t = last ? softmax(t) : relu(t);
        }
        return t;
    }
};

int main(int argc, char** argv) {
    if (argc != 5 && argc != 6) {
        fprintf(stderr, "usage: %s DATASET_DIR LAYERS HIDDEN EPOCHS [single|hybrid|model]\n", argv[0]);
        return 2;
    }
    const std::string engine_name = argc == 6 ? argv[5] : "single";
    if (engine_name != "single" && engine_name != "hybrid" && engine_name != "model") {
        fprintf(stderr, "unknown engine %s\n", engine_name.c_str());
        return 2;
    }
    const std::string dir = argv[1];
    const int layers = atoi(argv[2]), hidden = atoi(argv[3]), epochs = atoi(argv[4]);
    if (layers < 1 || hidden < 1 || epochs < 6) {
        fprintf(stderr, "need LAYERS >= 1, HIDDEN >= 1, EPOCHS >= 6 (the engine excludes five warm-up epochs)\n");
        return 2;
    }
    Context::init_context();

    CUDAStructualGraphLoader structure_loader;
    GraphNonStructualDataLoaderFullyReplicated data_loader;
    CUDAFullyStructualGraph* graph = structure_loader.load_graph_structure(
        dir + "/meta_data.txt", dir + "/edge_list.txt", dir + "/vertex_structure_partition.txt");
    AbstractGraphNonStructualData* data = data_loader.load_graph_non_structural_data(
        dir + "/meta_data.txt", dir + "/feature.txt", dir + "/label.txt", dir + "/vertex_data_partition.txt");
    graph->SetCuda(true);
    graph->InitMemory();
    graph->InitCsrBuffer();
    const int classes = data->get_num_labels();
    const int features = data->get_num_feature_dimensions();
    printf("driver: %u vertices, %d features, %d classes, %d layers, %d hidden units, %d epochs\n",
           (unsigned)graph->get_num_global_vertices(), features, classes, layers, hidden, epochs);

    DriverGCN* gcn = new DriverGCN(layers, hidden, classes, features);
    const int rank = DistributedSys::get_instance()->get_node_id();
    const int world = DistributedSys::get_instance()->get_num_nodes();
    SingleNodeExecutionEngineGPU* engine = NULL;
    ncclComm_t comm;
    if (engine_name == "single") {
        engine = new SingleNodeExecutionEngineGPU();
    } else if (engine_name == "hybrid") {
        engine = new DistributedPIPHybridParallelExecutionEngineGPU();
    } else {
        ncclUniqueId id;
        if (rank == 0) ncclGetUniqueId(&id);
        MPI_Bcast((void*)&id, sizeof(id), MPI_BYTE, 0, MPI_COMM_WORLD);
        ncclCommInitRank(&comm, world, id, rank);
        DistributedModelParallelExecutionEngineGPU* mp = new DistributedModelParallelExecutionEngineGPU();
        mp->SetNCCL(&comm, rank);
        engine = mp;
    }
    AdamOptimizerGPU* optimizer = new AdamOptimizerGPU(0.01, 0);
    // a scheduler that never fires (patience far beyond the run): the engine requires one
    LearningRateScheduler* scheduler = new LearningRateScheduler(0.01, 0.01, 0.8, 1e-8, 1 << 30, 0);
    OperatorExecutorGPUV2* executor = new OperatorExecutorGPUV2(graph);
    cublasHandle_t cublas;
    cudnnHandle_t cudnn;
    cusparseHandle_t cusparse;
    cublasCreate(&cublas);
    cudnnCreate(&cudnn);
    cusparseCreate(&cusparse);
    executor->set_activation_size(hidden, classes);
    executor->set_cuda_handle(&cublas, &cudnn, &cusparse);
    executor->build_inner_csr_();
    CrossEntropyLossGPU* loss = new CrossEntropyLossGPU();
    loss->set_elements_(graph->get_num_global_vertices(), classes);
    engine->setCuda(cudnn, graph->get_num_global_vertices());
    engine->set_graph_structure(graph);
    engine->set_graph_non_structural_data(data);
    engine->set_optimizer(optimizer);
    engine->set_operator_executor(executor);
    engine->set_loss(loss);
    engine->set_lr_scheduler(scheduler);

    const double acc = engine->execute_application(gcn, epochs);
    printf("driver: final accuracy %.4f\n", acc);
    fflush(stdout);
    Context::finalize_context();
    return 0;
}
