/*
 * make_checkpoint.cpp -- FIXTURE GENERATOR (test infrastructure): minml's own, unmodified host code and CPU backend write
 * a small network file in minml's on-disk format (Graph::save + FileSaver: a Json description, a newline, the binary
 * blob; optionally zlib-compressed as a whole) together with a seeded input and the outputs minml's CPU backend computes
 * for it (same container, tensors "input", "policy", "value"). The files it writes are committed next to this source; tests compare the checkpoint reader and the GPU path
 * against them.
 *
 * Built by `make -C oracle checkpoint_fixture` against the reference checkout, run as
 *     oracle/_ref/make_checkpoint tests/golden
 * Topology (the trunk's layer kinds at toy size, 9x9 board, 4 planes, 16 channels, batch 3):
 *     input -> conv3x3+relu -> batchnorm(relu) -> [conv3x3+relu -> conv3x3 -> add(relu)] x 2
 *           -> policy: conv1x1 -> softmax       -> value: global average pooling -> dense 3 -> softmax
 */
#include <minml/core/Context.hpp>
#include <minml/core/Device.hpp>
#include <minml/core/Shape.hpp>
#include <minml/core/Tensor.hpp>
#include <minml/graph/Graph.hpp>
#include <minml/graph/graph_optimizers.hpp>
#include <minml/layers/Add.hpp>
#include <minml/layers/BatchNormalization.hpp>
#include <minml/layers/Conv2D.hpp>
#include <minml/layers/Dense.hpp>
#include <minml/layers/GlobalAveragePooling.hpp>
#include <minml/layers/Softmax.hpp>
#include <minml/utils/file_util.hpp>
#include <minml/utils/json.hpp>
#include <minml/utils/serialization.hpp>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

using namespace ml;

static void randomize(Tensor &t, std::mt19937 &rng, float lo, float hi)
{
	std::uniform_real_distribution<float> dist(lo, hi);
	std::vector<float> tmp(t.volume());
	for (float &v : tmp)
		v = dist(rng);
	t.copyFromHost(tmp.data(), sizeof(float) * tmp.size());
}

int main(int argc, char *argv[])
{
	const std::string dir = argc > 1 ? argv[1] : ".";
	const int batch = 3, size = 9, planes = 4, channels = 16;

	Graph g;
	auto x = g.addInput(Shape( { batch, size, size, planes }));
	auto y = g.add(Conv2D(channels, 3, "linear").useBias(false), x);
	y = g.add(BatchNormalization("relu"), y);
	for (int i = 0; i < 2; i++)
	{
		auto t = g.add(Conv2D(channels, 3, "relu"), y);
		t = g.add(Conv2D(channels, 3, "linear"), t);
		y = g.add(Add("relu"), { t, y });
	}
	auto policy = g.add(Conv2D(1, 1, "linear"), y);
	policy = g.add(Softmax( { 1, 2, 3 }), policy);
	auto value = g.add(GlobalAveragePooling(), y);
	value = g.add(Dense(3, "linear"), value);
	value = g.add(Softmax( { 1 }), value);
	g.addOutput(policy);
	g.addOutput(value);
	g.init();

	// batch-norm statistics and biases that are not the freshly initialised zeros / ones
	std::mt19937 rng(20240607);
	for (int i = 0; i < g.numberOfNodes(); i++)
	{
		Layer &layer = g.getNode(i).getLayer();
		if (layer.name() == "BatchNormalization")
		{
			randomize(layer.getWeights().getParam(), rng, 0.5f, 1.5f); // gamma
			randomize(layer.getBias().getParam(), rng, -0.2f, 0.2f); // beta
			// the running mean (row 0) and variance (row 1) are private to the layer: hand them over the way a file would
			Tensor avg_var(Shape( { 2, channels }), DataType::FLOAT32, Device::cpu());
			std::vector<float> stats(2 * channels);
			std::uniform_real_distribution<float> mean(-0.5f, 0.5f), variance(0.5f, 1.5f);
			for (int c = 0; c < channels; c++)
			{
				stats[c] = mean(rng);
				stats[channels + c] = variance(rng);
			}
			avg_var.copyFromHost(stats.data(), sizeof(float) * stats.size());
			SerializedObject blob;
			Json params;
			params["avg_var"] = avg_var.serialize(blob);
			layer.loadParameters(params, blob);
		}
		else if (layer.getBias().getParam().volume() > 0)
			randomize(layer.getBias().getParam(), rng, -0.1f, 0.1f);
		if (layer.name() == "Conv2D" or layer.name() == "Dense")
		{ // He-uniform trunk weights; heads large enough that the softmax outputs are far from uniform
			Tensor &w = layer.getWeights().getParam();
			const bool head = w.dim(0) <= 3;
			const float limit = head ? 1.0f : std::sqrt(6.0f / (w.volume() / w.dim(0)));
			randomize(w, rng, -limit, limit);
		}
	}
	g.makeTrainable(false);

	SerializedObject binary;
	const Json description = g.save(binary);
	{
		FileSaver fs(dir + "/toy_network.bin");
		fs.save(description, binary, 2, false);
	}
	{
		FileSaver fs(dir + "/toy_network_compressed.bin");
		fs.save(description, binary, -1, true);
	}

	// minml's CPU dispatcher has no batch-norm inference (the call is commented out in src/core/math.cpp:727-729): networks
	// are folded before they are run. The file above keeps the layer; the outputs below come from the folded graph.
	FoldBatchNorm().optimize(g);

	std::vector<float> input(static_cast<size_t>(batch) * size * size * planes);
	for (float &v : input)
		v = (rng() % 10) < 3 ? 1.0f : 0.0f;
	g.getInput().copyFromHost(input.data(), sizeof(float) * input.size());
	g.predict(batch);
	g.context().synchronize();

	if (std::getenv("CHECKPOINT_DEBUG") != nullptr)
		for (int i = 0; i < g.numberOfNodes(); i++)
		{
			const Tensor &t = g.getNode(i).getOutputTensor();
			double sum = 0.0;
			for (int j = 0; j < t.volume(); j++)
				sum += std::fabs(reinterpret_cast<const float*>(t.data())[j]);
			std::printf("node %d %s: mean |x| = %g\n", i, g.getNode(i).getLayer().name().c_str(), sum / t.volume());
		}
	// input and outputs in the same container format, fp32 values in the blob
	SerializedObject io_binary;
	Json io;
	io["input"] = g.getInput().serialize(io_binary);
	io["policy"] = g.getOutput(0).serialize(io_binary);
	io["value"] = g.getOutput(1).serialize(io_binary);
	{
		FileSaver fs(dir + "/toy_network_io.bin");
		fs.save(io, io_binary, -1, false);
	}
	std::printf("wrote %s/toy_network{.bin,_compressed.bin,_io.bin}: %d nodes, %zu bytes of parameters\n", dir.c_str(), g.numberOfNodes(),
			binary.size());
	return 0;
}
