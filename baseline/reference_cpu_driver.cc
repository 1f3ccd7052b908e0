// Driver for the reference's single-node CPU engine, written against its public API (the call sequence of its own
// tests/test_single_node_training.cc, where dataset, model, loss and optimiser are hard-coded).  Nothing of the
// reference is modified; this main only chooses among the classes the reference ships:
//
//   reference_cpu_driver DATASET_DIR ORDER LAYERS HIDDEN EPOCHS LOSS OPTIMIZER LR [ENGINE]
//     ORDER     fc   : per layer weight, matmul, aggregation (applications/gcn.cc)
//               agg  : per layer aggregation, weight, matmul (tests/test_single_node_training.cc)
//     LOSS      ce | mse            (CrossEntropyLossCPU | MSELossCPU)
//     OPTIMIZER adam | sgd          (AdamOptimizerCPU(lr, 0) | SGDOptimizerCPU(lr))
//     ENGINE    single (default) | model | pipeline | chunked | mixed | hybrid - the reference's CPU engines; all but
//               "single" are multi-rank and are started with baseline/shims/mpirun_local.py (hybrid: exactly 4 ranks)
//
// The engines print one "Epoch e: Loss l, Accuracy a" line per epoch (rank 0); those lines are the golden curves.
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
#include "parallel/hybrid_parallel.h"
#include "parallel/model_parallel.h"
#include "parallel/pipelined_model_parallel.h"

class DriverGCN : public AbstractApplication {
    bool agg_first_;
    int layers_, hidden_, classes_;

  public:
    DriverGCN(bool agg_first, int layers, int hidden, int classes, int features)
        : AbstractApplication(features), agg_first_(agg_first), layers_(layers), hidden_(hidden), classes_(classes) {}
    Tensor* forward(Tensor* input) {
        Tensor* t = input;
        for (int i = 0; i < layers_; ++i) {
            const bool last = i == layers_ - 1;
            if (agg_first_) t = aggregation(t, NORM_SUM);
            Tensor* w = weight(t->dims[1], last ? classes_ : hidden_);
            t = matmul(t, w);
            if (!agg_first_) t = aggregation(t, NORM_SUM);
            t = last ? softmax(t) : relu(t);
        }
        return t;
    }
};

int main(int argc, char** argv) {
    if (argc != 9 && argc != 10) {
        fprintf(stderr, "usage: %s DATASET_DIR fc|agg LAYERS HIDDEN EPOCHS ce|mse adam|sgd LR [single|model|pipeline|chunked|mixed|hybrid]\n", argv[0]);
        return 2;
    }
    const std::string engine_name = argc == 10 ? argv[9] : "single";
    const std::string dir = argv[1], order = argv[2], loss_name = argv[6], opt_name = argv[7];
    const int layers = atoi(argv[3]), hidden = atoi(argv[4]), epochs = atoi(argv[5]);
    const double lr = atof(argv[8]);
    if ((order != "fc" && order != "agg") || (loss_name != "ce" && loss_name != "mse") || (opt_name != "adam" && opt_name != "sgd") ||
        layers < 1 || hidden < 1 || epochs < 6 || !(lr > 0)) {
        fprintf(stderr, "bad arguments (EPOCHS >= 6: the engine excludes five warm-up epochs from its timing)\n");
        return 2;
    }
    Context::init_context();
    GraphStructureLoaderFullyReplicated structure_loader;
    GraphNonStructualDataLoaderFullyReplicated data_loader;
    AbstractGraphStructure* graph = structure_loader.load_graph_structure(
        dir + "/meta_data.txt", dir + "/edge_list.txt", dir + "/vertex_structure_partition.txt");
    AbstractGraphNonStructualData* data = data_loader.load_graph_non_structural_data(
        dir + "/meta_data.txt", dir + "/feature.txt", dir + "/label.txt", dir + "/vertex_data_partition.txt");
    DriverGCN* gcn = new DriverGCN(order == "agg", layers, hidden, data->get_num_labels(), data->get_num_feature_dimensions());
    AbstractExecutionEngine* engine = NULL;
    if (engine_name == "single") engine = new SingleNodeExecutionEngineCPU();
    else if (engine_name == "model") engine = new DistributedModelParallelExecutionEngineCPU();
    else if (engine_name == "pipeline") engine = new DistributedPipelinedLinearModelParallelExecutionEngineCPU();
    else if (engine_name == "chunked") engine = new DistributedPipelinedLinearModelParallelWithGraphChunkingExecutionEngineCPU();
    else if (engine_name == "mixed") engine = new MixedDistributedPipelinedLinearModelParallelWithGraphChunkingExecutionEngineCPU();
    else if (engine_name == "hybrid") engine = new DistributedPIPHybridParallelExecutionEngineCPU();
    else { fprintf(stderr, "unknown engine %s\n", engine_name.c_str()); return 2; }
    AbstractOptimizer* optimizer = opt_name == "adam" ? (AbstractOptimizer*)new AdamOptimizerCPU(lr, 0.0) : (AbstractOptimizer*)new SGDOptimizerCPU(lr);
    AbstractOperatorExecutor* executor = new OperatorExecutorCPU(graph);
    AbstractLoss* loss = loss_name == "ce" ? (AbstractLoss*)new CrossEntropyLossCPU() : (AbstractLoss*)new MSELossCPU();
    engine->set_graph_structure(graph);
    engine->set_graph_non_structural_data(data);
    engine->set_optimizer(optimizer);
    engine->set_operator_executor(executor);
    engine->set_loss(loss);
    const double acc = engine->execute_application(gcn, epochs);
    printf("driver: final accuracy %.4f\n", acc);
    fflush(stdout);
    Context::finalize_context();
    return 0;
}
