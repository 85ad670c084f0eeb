/*
 * make_calibration.cpp -- FIXTURE GENERATOR (test infrastructure): minml's own Histogram (src/graph/Histogram.cpp) collects
 * statistics of seeded activations until it declares itself ready, and its serialised state (range, bins, the int8
 * transform it derived) is written in minml's container format. tests/test_calibration.py regenerates the same activations
 * (the generator below uses only exactly reproducible fp32 arithmetic) and checks the Python restatement against this file.
 *
 * Built by `make -C oracle calibration_fixture` against the reference checkout, run as
 *     oracle/_ref/make_calibration tests/golden
 * Two histograms of 2048 bins, accuracy 0.01, 256 target bins:
 *     "relu"    activations after a ReLU (the hint fixes the lower end of the range at 0), with a heavy tail
 *     "linear"  signed activations without a hint (the range comes from the data until outliers are rare enough)
 */
#include <minml/core/Device.hpp>
#include <minml/core/Shape.hpp>
#include <minml/core/Tensor.hpp>
#include <minml/graph/Histogram.hpp>
#include <minml/layers/Layer.hpp>
#include <minml/utils/file_util.hpp>
#include <minml/utils/json.hpp>
#include <minml/utils/serialization.hpp>

#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

using namespace ml;

/* 64-bit linear congruential generator; a draw is the top 24 bits as a float in [0, 1) -- exact in fp32 */
struct Lcg
{
		uint64_t state;
		float uniform()
		{
			state = state * 6364136223846793005ull + 1442695040888963407ull;
			return static_cast<float>(state >> 40) * (1.0f / 16777216.0f);
		}
};
/* sum of four uniforms, centred: bell-shaped, only additions and multiplications (bit-identical in numpy fp32) */
static float bell(Lcg &g)
{
	const float a = g.uniform(), b = g.uniform(), c = g.uniform(), d = g.uniform();
	return ((a + b) + (c + d)) - 2.0f;
}
static void fill(std::vector<float> &batch, Lcg &g, bool relu)
{
	for (float &v : batch)
	{
		float x = bell(g) * 1.5f + 0.25f;
		if (g.uniform() < 0.015625f)
			x = x * 4.0f; // a heavy tail: 1 value in 64 is four times larger
		v = relu ? (x > 0.0f ? x : 0.0f) : x;
	}
}

int main(int argc, char *argv[])
{
	const std::string dir = argc > 1 ? argv[1] : ".";
	const int rows = 32, cols = 64, max_batches = 400;
	SerializedObject binary;
	Json description;
	for (int which = 0; which < 2; which++)
	{
		const bool relu = (which == 0);
		Histogram h(2048, 0.01f, 256);
		if (relu)
			h.setHint(ActivationType::RELU);
		Lcg g { relu ? 12345ull : 67890ull };
		Tensor t(Shape( { rows, cols }), DataType::FLOAT32, Device::cpu());
		std::vector<float> batch(rows * cols);
		int batches = 0;
		while (not h.isReady() and batches < max_batches)
		{
			fill(batch, g, relu);
			t.copyFromHost(batch.data(), sizeof(float) * batch.size());
			h.collectStatistics(t);
			batches++;
		}
		Json entry = h.serialize(binary);
		entry["batches"] = batches;
		entry["rows"] = rows;
		entry["cols"] = cols;
		entry["seed"] = relu ? 12345 : 67890;
		entry["bins"] = 2048;
		description[relu ? "relu" : "linear"] = entry;
		std::printf("%s: %d batches, %s\n", relu ? "relu" : "linear", batches, h.getInfo().c_str());
	}
	FileSaver fs(dir + "/calibration_histograms.bin");
	fs.save(description, binary, 2, false);
	return 0;
}
