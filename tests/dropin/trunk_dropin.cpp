/*
 * trunk_dropin.cpp -- TEST PROGRAM: minml's own, unmodified host code (Graph, Conv2D, Dense, Add, GlobalAveragePooling,
 * core/math.cpp dispatcher, Tensor, Context) driving libminml_b200.so as its CUDA backend.
 *
 * It is compiled against the reference's headers and linked with the reference's host sources (built in place from the
 * reference checkout by oracle/Makefile, target `dropin`) and with libminml_b200.so in place of src/backend/cuda.
 * It builds the ResNet-trunk topology through minml's public Graph API, runs it on Device::cpu() in fp32 and on
 * Device::cuda(0) in fp16 (or fp32) from the same parameters and input, and prints the largest difference relative to the
 * largest reference value for each output as one JSON line.
 *
 *   trunk_dropin <batch> <height> <width> <planes> <channels> <blocks> <fp16|fp32> [repeats]
 *
 * With DROPIN_TIMING_ONLY=1 in the environment the CPU run and the comparison are skipped (the error fields read -1): the
 * program then only times `repeats` calls of Graph::predict on the device after three warm-up calls, which is how bench.py
 * measures the throughput of the library under minml's own host loop at the full benchmark batch sizes.
 */
#include <minml/core/Context.hpp>
#include <minml/core/Device.hpp>
#include <minml/core/Shape.hpp>
#include <minml/core/Tensor.hpp>
#include <minml/graph/Graph.hpp>
#include <minml/graph/graph_optimizers.hpp>
#include <minml/layers/Add.hpp>
#include <minml/layers/Conv2D.hpp>
#include <minml/layers/Dense.hpp>
#include <minml/layers/GlobalAveragePooling.hpp>
#include <minml/utils/json.hpp>
#include <minml/utils/serialization.hpp>

#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

using namespace ml;

static void on_crash(int sig)
{ // a crash in host code prints where it happened (function names only) instead of dying silently
	void *frames[64];
	const int n = backtrace(frames, 64);
	const char msg[] = "trunk_dropin: fatal signal, backtrace follows\n";
	(void) !write(2, msg, sizeof(msg) - 1);
	backtrace_symbols_fd(frames, n, 2);
	_exit(128 + sig);
}
static void stage(const char *what)
{
	if (std::getenv("DROPIN_VERBOSE") != nullptr)
		std::fprintf(stderr, "[trunk_dropin] %s\n", what);
}

static void build(Graph &g, int batch, int h, int w, int planes, int channels, int blocks)
{
	auto x = g.addInput(Shape( { batch, h, w, planes }));
	auto y = g.add(Conv2D(channels, 3, "relu"), x);
	for (int i = 0; i < blocks; i++)
	{
		auto t = g.add(Conv2D(channels, 3, "relu"), y);
		t = g.add(Conv2D(channels, 3, "linear"), t);
		y = g.add(Add("relu"), { t, y });
	}
	auto policy = g.add(Conv2D(1, 1, "linear"), y);
	auto pooled = g.add(GlobalAveragePooling(), y);
	auto value = g.add(Dense(3, "linear"), pooled);
	g.addOutput(policy);
	g.addOutput(value);
	g.init();
}

static std::vector<float> to_host_fp32(Graph &g, int index)
{
	Tensor out = g.getOutput(index); // a view sharing the data
	Tensor tmp(out.shape(), out.dtype(), Device::cpu());
	tmp.copyFrom(g.context(), out);
	g.context().synchronize();
	Context cpu_ctx;
	tmp.convertTo(cpu_ctx, DataType::FLOAT32);
	std::vector<float> result(tmp.volume());
	std::memcpy(result.data(), tmp.data(), sizeof(float) * result.size());
	return result;
}

int main(int argc, char *argv[])
{
	signal(SIGSEGV, on_crash);
	signal(SIGABRT, on_crash);
	if (argc < 8)
	{
		std::fprintf(stderr, "usage: %s batch height width planes channels blocks fp16|fp32 [repeats]\n", argv[0]);
		return 2;
	}
	const int batch = std::atoi(argv[1]), h = std::atoi(argv[2]), w = std::atoi(argv[3]), planes = std::atoi(argv[4]);
	const int channels = std::atoi(argv[5]), blocks = std::atoi(argv[6]);
	const bool fp16 = std::strcmp(argv[7], "fp16") == 0;
	const int repeats = argc > 8 ? std::atoi(argv[8]) : 0;
	stage("build cpu graph");
	Graph cpu_graph;
	build(cpu_graph, batch, h, w, planes, channels, blocks);
	cpu_graph.makeTrainable(false); // Graph::save of a trainable graph wants an optimizer

	// the same parameters for the second graph, through minml's own serialisation (before the Add layers are folded away)
	stage("save / load");
	SerializedObject binary;
	const Json description = cpu_graph.save(binary);
	Graph gpu_graph;
	gpu_graph.load(description, binary);
	gpu_graph.makeTrainable(false);
	FoldAdd().optimize(cpu_graph);
	FoldAdd().optimize(gpu_graph);
	if (Device::numberOfCudaDevices() == 0)
	{
		std::printf("{\"error\": \"no CUDA device visible to the backend\"}\n");
		return 3;
	}
	stage("moveTo cuda");
	gpu_graph.moveTo(Device::cuda(0));
	stage("moved");
	if (fp16)
		gpu_graph.convertTo(DataType::FLOAT16);

	// Bernoulli(0.3) input planes
	stage("inputs");
	std::mt19937 rng(1234);
	std::vector<float> input(static_cast<size_t>(batch) * h * w * planes);
	for (float &v : input)
		v = (rng() % 10) < 3 ? 1.0f : 0.0f;
	cpu_graph.getInput().copyFromHost(input.data(), sizeof(float) * input.size());
	{
		Tensor staged(Shape( { batch, h, w, planes }), DataType::FLOAT32, Device::cpu());
		staged.copyFromHost(input.data(), sizeof(float) * input.size());
		if (fp16)
		{
			Context cpu_ctx;
			staged.convertTo(cpu_ctx, DataType::FLOAT16);
		}
		gpu_graph.getInput().copyFrom(gpu_graph.context(), staged);
	}

	const bool timing_only = std::getenv("DROPIN_TIMING_ONLY") != nullptr && std::getenv("DROPIN_TIMING_ONLY")[0] == '1';
	if (not timing_only)
	{
		stage("predict cpu");
		cpu_graph.predict(batch);
		cpu_graph.context().synchronize();
	}
	stage("predict cuda");
	for (int i = 0; i < (timing_only ? 3 : 1); i++)
		gpu_graph.predict(batch);
	gpu_graph.context().synchronize();
	stage("predicted");

	double seconds = 0.0;
	if (repeats > 0)
	{
		const auto t0 = std::chrono::steady_clock::now();
		for (int i = 0; i < repeats; i++)
			gpu_graph.predict(batch);
		gpu_graph.context().synchronize();
		seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
	}

	double rel[2] = { -1.0, -1.0 };
	for (int o = 0; o < 2 and not timing_only; o++)
	{
		std::vector<float> want(cpu_graph.getOutput(o).volume());
		std::memcpy(want.data(), cpu_graph.getOutput(o).data(), sizeof(float) * want.size());
		const std::vector<float> got = to_host_fp32(gpu_graph, o);
		double max_ref = 0.0, max_diff = 0.0;
		for (size_t i = 0; i < want.size(); i++)
		{
			max_ref = std::max(max_ref, std::fabs(static_cast<double>(want[i])));
			max_diff = std::max(max_diff, std::fabs(static_cast<double>(want[i]) - got[i]));
		}
		rel[o] = max_diff / std::max(max_ref, 1e-30);
	}
	std::printf("{\"nodes\": %d, \"policy_rel_err\": %.6g, \"value_rel_err\": %.6g, \"positions_per_s\": %.1f}\n", gpu_graph.numberOfNodes(), rel[0],
			rel[1], repeats > 0 ? batch * repeats / seconds : 0.0);
	return 0;
}
