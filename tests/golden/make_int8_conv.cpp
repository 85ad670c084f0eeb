/*
 * make_int8_conv.cpp -- FIXTURE GENERATOR (test infrastructure): minml's own, unmodified Conv2D layer quantises seeded fp32
 * weights (Layer::setupQuantization -> quantize_weights, src/layers/Layer.cpp:147-160, src/layers/quantization.cpp:59-97) and
 * runs its integer forward pass on Device::cpu() -- the scalar loop of src/layers/Conv2D.cpp:240-308, which is the definition
 * of the int32 accumulators, of the padding with the quantised zero and of the requantisation order.  Inputs, quantised
 * parameters and outputs of every case are written in minml's container format (Json description, newline, binary blob);
 * tests/test_oracle.py holds the C restatement (oracle/oracle.c) to these outputs bit for bit, and the GPU tests hold the
 * fused and the three-call int8 paths to the same file.
 *
 * Built by `make -C oracle int8_fixture` against the reference checkout, run as
 *     oracle/_ref/make_int8_conv tests/golden
 * Cases (36 input and 44 output channels on a 12 x 13 board unless the name says otherwise: the channel counts of the
 * reference's own int8 test, test/backend/test_quantization.cpp:173-240):
 *     k3_relu_ext_i8      3x3, ReLU, residual input, asymmetric input transform (quantised zero -37), int8 output
 *     k3_linear_f32       3x3, linear, no residual, asymmetric input transform (quantised zero 55), fp32 output
 *     k3_tanh_sym_i8      3x3, tanh, residual, symmetric transforms (quantised zero 0), int8 output
 *     k3_relu_min_i8      3x3, ReLU, residual, quantised zero -128 (what a histogram calibrator yields after a ReLU), int8 output
 *     k1_sigmoid_ext_i8   1x1, sigmoid, residual, asymmetric input transform, int8 output
 *     k3_relu_ext_i8_c32  as the first, 32 -> 48 channels (a channel count the fused gather kernel accepts)
 *     k3_relu_ext_i8_c128 as the fourth, 128 -> 64 channels on a 6 x 7 board (the fused kernel's copy-engine operand path with its
 *                         border corrections for the non-zero quantised zero)
 *     k3_linear_f32_c128  as the second, 128 -> 64 channels on a 6 x 7 board
 */
#include <minml/core/Context.hpp>
#include <minml/core/Device.hpp>
#include <minml/core/Shape.hpp>
#include <minml/core/Tensor.hpp>
#include <minml/layers/Conv2D.hpp>
#include <minml/layers/quantization.hpp>
#include <minml/utils/file_util.hpp>
#include <minml/utils/json.hpp>
#include <minml/utils/serialization.hpp>

#include <cstdint>
#include <cstdio>
#include <memory>
#include <random>
#include <string>
#include <vector>

using namespace ml;

struct Case
{
		const char *name;
		int batch, height, width, cin, cout, kernel;
		const char *activation;
		bool with_ext, int8_output;
		float in_scale, in_shift, ext_scale, ext_shift, out_scale, out_shift;
};

static Tensor int8_tensor(const Shape &shape, std::mt19937 &rng, int lo, int hi)
{
	Tensor t(shape, DataType::INT8, Device::cpu());
	std::vector<int8_t> tmp(t.volume());
	std::uniform_int_distribution<int> dist(lo, hi);
	for (int8_t &v : tmp)
		v = static_cast<int8_t>(dist(rng));
	t.copyFromHost(tmp.data(), tmp.size());
	return t;
}
static void fill_normal(Tensor &t, std::mt19937 &rng, float stddev)
{
	std::normal_distribution<float> dist(0.0f, stddev);
	std::vector<float> tmp(t.volume());
	for (float &v : tmp)
		v = dist(rng);
	t.copyFromHost(tmp.data(), sizeof(float) * tmp.size());
}
/* (scale, shift) pairs go into the blob as fp32: the Json writer keeps six decimals only */
static Json transforms_json(const Case &c, SerializedObject &binary)
{
	const float values[6] = { c.in_scale, c.in_shift, c.ext_scale, c.ext_shift, c.out_scale, c.out_shift };
	Tensor t(Shape( { 3, 2 }), DataType::FLOAT32, Device::cpu());
	t.copyFromHost(values, sizeof(values));
	return t.serialize(binary);
}

int main(int argc, char *argv[])
{
	const std::string dir = argc > 1 ? argv[1] : ".";
	// a transform t maps int8 q to the real value q * scale + shift; its quantised zero is round(-shift / scale)
	const Case cases[] = {
			{ "k3_relu_ext_i8", 3, 12, 13, 36, 44, 3, "relu", true, true, 0.02f, 0.74f, 0.03f, -0.45f, 0.025f, 1.1f },
			{ "k3_linear_f32", 2, 12, 13, 36, 44, 3, "linear", false, false, 0.015f, -0.825f, 1.0f, 0.0f, 1.0f, 0.0f },
			{ "k3_tanh_sym_i8", 2, 12, 13, 36, 44, 3, "tanh", true, true, 0.02f, 0.0f, 0.01f, 0.0f, 0.0078125f, 0.0f },
			{ "k3_relu_min_i8", 2, 12, 13, 36, 44, 3, "relu", true, true, 0.0125f, 1.6f, 0.02f, 2.56f, 0.03f, 3.84f },
			{ "k1_sigmoid_ext_i8", 5, 12, 13, 36, 44, 1, "sigmoid", true, true, 0.03f, 0.21f, 0.04f, 0.3f, 0.00390625f, 0.5f },
			{ "k3_relu_ext_i8_c32", 2, 12, 13, 32, 48, 3, "relu", true, true, 0.02f, 0.74f, 0.03f, -0.45f, 0.025f, 1.1f },
			{ "k3_relu_ext_i8_c128", 2, 6, 7, 128, 64, 3, "relu", true, true, 0.0125f, 1.6f, 0.02f, 2.56f, 0.03f, 3.84f },
			{ "k3_linear_f32_c128", 1, 6, 7, 128, 64, 3, "linear", false, false, 0.015f, -0.825f, 1.0f, 0.0f, 1.0f, 0.0f } };

	SerializedObject binary;
	Json description;
	std::mt19937 rng(20250206);
	for (const Case &c : cases)
	{
		std::shared_ptr<Context> context = std::make_shared<Context>(Device::cpu());
		const int cin = c.cin, cout = c.cout;
		Conv2D layer(cout, c.kernel, c.activation);
		const Shape in_shape( { c.batch, c.height, c.width, cin });
		const Shape out_shape( { c.batch, c.height, c.width, cout });
		if (c.with_ext)
			layer.setInputShape(std::vector<Shape> { in_shape, out_shape });
		else
			layer.setInputShape(std::vector<Shape> { in_shape });
		layer.changeContext(context);
		fill_normal(layer.getWeights().getParam(), rng, std::sqrt(2.0f / (c.kernel * c.kernel * cin)));
		fill_normal(layer.getBias().getParam(), rng, 0.05f);

		Json entry;
		entry["name"] = c.name;
		entry["kernel"] = c.kernel;
		entry["activation"] = c.activation;
		entry["transforms"] = transforms_json(c, binary); // [input, ext, output] x [scale, shift]
		// the fp32 parameters before quantisation (left out where they would dominate the file: the wide cases)
		const bool keep_raw = cin < 128;
		entry["raw_weights"] = keep_raw ? layer.getWeights().getParam().serialize(binary) : Json::null();
		entry["raw_bias"] = keep_raw ? layer.getBias().getParam().serialize(binary) : Json::null();

		std::vector<AffineTransform> input_transforms { AffineTransform(c.in_scale, c.in_shift) };
		if (c.with_ext)
			input_transforms.push_back(AffineTransform(c.ext_scale, c.ext_shift));
		layer.setupQuantization(input_transforms, AffineTransform(c.out_scale, c.out_shift), 8);
		if (c.int8_output)
			layer.convertTo(DataType::INT8); // what the Quantize pass does when every consumer is quantised too
		entry["input_zero"] = static_cast<int>(get_zero<int32_t>(input_transforms[0]));

		std::vector<Tensor> inputs { int8_tensor(in_shape, rng, -128, 127) };
		if (c.with_ext)
			inputs.push_back(int8_tensor(out_shape, rng, -128, 127));
		Tensor output(out_shape, c.int8_output ? DataType::INT8 : DataType::FLOAT32, Device::cpu());
		layer.forward(inputs, output);
		context->synchronize();

		entry["weights"] = layer.getWeights().getParam().serialize(binary);
		entry["bias"] = layer.getBias().getParam().serialize(binary);
		{ // the channel scales are reachable only through saveParameters, which also writes weights and bias: use a scratch blob
			SerializedObject scratch;
			const Json params = layer.saveParameters(scratch);
			Tensor channel_scales;
			channel_scales.unserialize(params["channel_scales"], scratch);
			entry["channel_scales"] = channel_scales.serialize(binary);
		}
		entry["input"] = inputs[0].serialize(binary);
		entry["ext"] = c.with_ext ? inputs[1].serialize(binary) : Json::null();
		entry["output"] = output.serialize(binary);
		description[c.name] = entry;
		std::printf("%s: done\n", c.name);
	}
	FileSaver fs(dir + "/int8_conv_cases.bin");
	fs.save(description, binary, -1, false);
	return 0;
}
