/*
 * make_checkpoint.cpp -- FIXTURE GENERATOR (test infrastructure): minml's own, unmodified host code and CPU backend write
 * a small network file in minml's on-disk format (Graph::save + FileSaver: a Json description, a newline, the binary
 * blob; optionally zlib-compressed as a whole) together with a seeded input and the outputs minml's CPU backend computes
 * for it (same container, tensors "input", "policy", "value"). The files it writes are committed next to this source; tests compare the checkpoint reader and the GPU path
 * against them.
 *
 * Built by `make -C oracle checkpoint_fixture` against the reference checkout, run as
 *     oracle/_ref/make_checkpoint tests/golden
 * toy_network: the trunk's layer kinds at toy size (9x9 board, 4 planes, 16 channels, batch 3):
 *     input -> conv3x3+relu -> batchnorm(relu) -> [conv3x3+relu -> conv3x3 -> add(relu)] x 2
 *           -> policy: conv1x1 -> softmax       -> value: global average pooling -> dense 3 -> softmax
 * toy_block_network: the block of minml's current architectures (12x12 board, 4 planes, batch 2):
 *     input -> space-to-depth 2x2 -> conv1x1 32 +relu
 *           -> [depthwise 7x7 -> RMS norm -> conv1x1+relu -> conv1x1 -> squeeze-and-excitation (pooling, dense 8 relu, dense 32
 *               sigmoid, channel scaling) -> add] -> policy: depth-to-space 2x2 -> conv1x1 -> softmax; value as above
 */
#include <minml/core/Context.hpp>
#include <minml/core/Device.hpp>
#include <minml/core/Shape.hpp>
#include <minml/core/Tensor.hpp>
#include <minml/graph/Graph.hpp>
#include <minml/graph/graph_optimizers.hpp>
#include <minml/layers/Add.hpp>
#include <minml/layers/BatchNormalization.hpp>
#include <minml/layers/ChannelScaling.hpp>
#include <minml/layers/Conv2D.hpp>
#include <minml/layers/Dense.hpp>
#include <minml/layers/DepthToSpace.hpp>
#include <minml/layers/DepthwiseConv2D.hpp>
#include <minml/layers/GlobalAveragePooling.hpp>
#include <minml/layers/RMSNormalization.hpp>
#include <minml/layers/Softmax.hpp>
#include <minml/layers/SpaceToDepth.hpp>
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

	/* ---- the second network */
	{
		const int b2 = 2, board = 12, ch = 32;
		Graph g2;
		auto in = g2.addInput(Shape( { b2, board, board, planes }));
		auto y2 = g2.add(SpaceToDepth(2), in);
		y2 = g2.add(Conv2D(ch, 1, "relu"), y2);
		auto t = g2.add(DepthwiseConv2D(ch, 7), y2);
		t = g2.add(RMSNormalization(), t);
		t = g2.add(Conv2D(ch, 1, "relu"), t);
		t = g2.add(Conv2D(ch, 1, "linear"), t);
		auto se = g2.add(GlobalAveragePooling(), t);
		se = g2.add(Dense(8, "relu"), se);
		se = g2.add(Dense(ch, "sigmoid"), se);
		t = g2.add(ChannelScaling(), { t, se });
		y2 = g2.add(Add("linear"), { t, y2 });
		auto p2 = g2.add(DepthToSpace(2, Shape( { board, board })), y2);
		p2 = g2.add(Conv2D(1, 1, "linear"), p2);
		p2 = g2.add(Softmax( { 1, 2, 3 }), p2);
		auto v2 = g2.add(GlobalAveragePooling(), y2);
		v2 = g2.add(Dense(3, "linear"), v2);
		v2 = g2.add(Softmax( { 1 }), v2);
		g2.addOutput(p2);
		g2.addOutput(v2);
		g2.init();
		for (int i = 0; i < g2.numberOfNodes(); i++)
		{
			Layer &layer = g2.getNode(i).getLayer();
			Tensor &w = layer.getWeights().getParam();
			if (layer.getBias().getParam().volume() > 0)
				randomize(layer.getBias().getParam(), rng, -0.1f, 0.1f);
			if (layer.name() == "Conv2D" or layer.name() == "Dense")
			{
				const bool head = w.dim(0) <= 3;
				const float limit = head ? 1.0f : std::sqrt(6.0f / (w.volume() / w.dim(0)));
				randomize(w, rng, -limit, limit);
			}
			else if (layer.name() == "DepthwiseConv2D")
				randomize(w, rng, -0.25f, 0.25f);
			else if (layer.name() == "RMSNormalization")
				randomize(w, rng, 0.5f, 1.5f);
		}
		g2.makeTrainable(false);
		SerializedObject binary2;
		const Json description2 = g2.save(binary2);
		{
			FileSaver fs(dir + "/toy_block_network.bin");
			fs.save(description2, binary2, 2, false);
		}
		std::vector<float> input2(static_cast<size_t>(b2) * board * board * planes);
		for (float &v : input2)
			v = (rng() % 10) < 3 ? 1.0f : 0.0f;
		g2.getInput().copyFromHost(input2.data(), sizeof(float) * input2.size());
		g2.predict(b2);
		g2.context().synchronize();
		SerializedObject io_binary2;
		Json io2;
		io2["input"] = g2.getInput().serialize(io_binary2);
		io2["policy"] = g2.getOutput(0).serialize(io_binary2);
		io2["value"] = g2.getOutput(1).serialize(io_binary2);
		FileSaver fs(dir + "/toy_block_network_io.bin");
		fs.save(io2, io_binary2, -1, false);
		std::printf("wrote %s/toy_block_network{.bin,_io.bin}: %d nodes, %zu bytes of parameters\n", dir.c_str(), g2.numberOfNodes(), binary2.size());
	}
	std::printf("wrote %s/toy_network{.bin,_compressed.bin,_io.bin}: %d nodes, %zu bytes of parameters\n", dir.c_str(), g.numberOfNodes(),
			binary.size());
	return 0;
}
