// Measurement harness around the UNMODIFIED reference (zhan-wei-919/llm), for the reference arm
// of bench.py.  It includes the reference's own headers from a copy of its tree (-I <copy>) and
// assembles the TinyLlama model exactly as the reference's programs do
// (model/llm/tiny_llama.cpp:25-71, model/llm/test/bench_tiny_llama_load.cu:30-52,162-186):
// modules, LLM, Engine, KV_Pool, load_safetensor, Scheduler, PipelineDriver, LLM::inference.
// Nothing of llm_b200 is compiled or linked in here.
//
//   ref_harness --weights model.safetensors [--max-seqs 8] [--max-tokens 512] [--max-seq-len 2048]
//               [--layers 22]
//
// Commands come one per line on standard input; each prints one JSON line:
//   decode B P W K      B requests with P-token prompts through the scheduler; after every request
//                       decodes, W warm-up steps, then K timed decode steps of the whole batch
//   prefill T W K       one request of T tokens as one step (needs --max-tokens >= T), W + K times
//   load R P N          the reference's own load benchmark: R requests, P prompt + N new tokens
//   logits FILE t0 t1.. one prompt as one step; the last row's logits (bf16 -> float32) to FILE
#include "model/modules/Attention.h"
#include "model/modules/Embedding.h"
#include "model/modules/LMHead.h"
#include "model/modules/MLP.h"
#include "model/modules/RMSNorm.h"
#include "model/modules/Residual.h"
#include "runtime/Driver.h"
#include "runtime/Engine.h"
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cuda_bf16.h>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

// Sizes of TinyLlama 1.1B (model/llm/tiny_llama.cpp:17-21); the attention kernel of the reference
// exists for exactly this head layout (kernel/attention/Attention.h:12-19).
constexpr int NH = 32, NKV = 4, HS = 64;
constexpr int HIDDEN = 2048, INTERMEDIATE = 5632, VOCAB = 32000;
constexpr float RMS_EPS = 1e-5f, ROPE_THETA = 10000.0f;

static int g_max_tokens = 512;

template<typename T>
class Block {
public:
	Block(LLM &llm, Engine &engine, Tensor *input, int layer)
	: input_norm_(llm, input, g_max_tokens, HIDDEN, RMS_EPS, prefix(layer) + ".input_layernorm")
	, self_attn_(llm, engine, input_norm_.out(), g_max_tokens, HIDDEN, layer, false, false, -1, prefix(layer) + ".self_attn")
	, attention_residual_(llm, input, self_attn_.out(), g_max_tokens, HIDDEN)
	, post_attention_norm_(llm, attention_residual_.out(), g_max_tokens, HIDDEN, RMS_EPS, prefix(layer) + ".post_attention_layernorm")
	, mlp_(llm, post_attention_norm_.out(), g_max_tokens, HIDDEN, INTERMEDIATE, false, prefix(layer) + ".mlp")
	, mlp_residual_(llm, attention_residual_.out(), mlp_.out(), g_max_tokens, HIDDEN) {}
	Tensor *out() {return mlp_residual_.out();}
private:
	static std::string prefix(int layer) {return "model.layers." + std::to_string(layer);}
	RMSNorm<T> input_norm_;
	Attention<T> self_attn_;
	Residual<T> attention_residual_;
	RMSNorm<T> post_attention_norm_;
	MLP<T> mlp_;
	Residual<T> mlp_residual_;
};

static uint64_t g_rng = 0x9E3779B97F4A7C15ull;
static int next_token() {
	g_rng = g_rng * 6364136223846793005ull + 1442695040888963407ull;
	return (int)((g_rng >> 33) % VOCAB);
}
static std::vector<int> random_prompt(int n) {
	std::vector<int> p(n);
	for (int &t : p) t = next_token();
	return p;
}

static double now_ms() {
	return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

static bool cuda_ok(const char *what) {
	cudaError_t e = cudaGetLastError();
	if (e == cudaSuccess) e = cudaDeviceSynchronize();
	if (e != cudaSuccess) {
		std::printf("{\"error\": \"%s: %s\"}\n", what, cudaGetErrorString(e));
		std::fflush(stdout);
		return false;
	}
	return true;
}

struct Harness {
	LLM &llm;
	Engine &engine;
	KV_Pool &pool;
	Tensor *logits;
	int max_seqs, max_tokens, max_seq_len;
	LLM::InferenceBuffers buffers;

	Harness(LLM &l, Engine &e, KV_Pool &p, Tensor *lg, int s, int t, int len)
	: llm(l), engine(e), pool(p), logits(lg), max_seqs(s), max_tokens(t), max_seq_len(len) {
		buffers.input_stride = max_tokens;
		buffers.token_stride = max_seqs;
		cudaHostAlloc(&buffers.h_inputs, 2 * buffers.input_stride * sizeof(int), 0);
		cudaMalloc(&buffers.d_tokens, 2 * buffers.token_stride * sizeof(int));
		cudaHostAlloc(&buffers.h_tokens, 2 * buffers.token_stride * sizeof(int), 0);
	}

	// bytes that one step copies to the device (token ids, LLM.h:210; metadata, Engine.h:109-116)
	// and back (the sampled tokens, LLM.h:218)
	long h2d_bytes(int B, int T) const {
		int W = pool.max_blocks_per_seq();
		return 4L * (T + (long)B * W + B + T + T + B + 1);
	}

	struct Step {cudaEvent_t start, end; bool timed;};

	// The reference's driver keeps two batches in flight (runtime/Driver.h:29-53), so B requests
	// that left their prompts at different times decode as two alternating groups; when all of
	// them leave in one step they decode as one batch that is waited for each step.  Either way
	// a "step" here is one new token for each of the B requests, counted from launched batches
	// in the steady state (every request decoding, none waiting for its prompt).
	void decode(int B, int P, int W, int K) {
		if (B > max_seqs || P > max_tokens || P + W + K + 64 > max_seq_len) {
			std::printf("{\"mode\": \"decode\", \"refused\": \"batch %d / prompt %d exceed --max-seqs %d / --max-tokens %d\"}\n", B, P, max_seqs, max_tokens);
			return;
		}
		LocalKvHandoff handoff;
		Scheduler scheduler(pool, {max_seqs, max_tokens, /*eos=*/-1}, handoff);
		int per_step = std::max(1, max_tokens / P);
		int prefill_steps = (B + per_step - 1) / per_step;
		int max_new = prefill_steps + W + K + 8;
		for (int r = 0; r < B; ++r) scheduler.add_request(random_prompt(P), max_new);
		std::vector<Step> steps;
		steps.reserve(4 * (max_new + prefill_steps) + 16);
		long steady_tokens = 0, window_tokens = 0, window_h2d = 0;
		int prompts_done = 0, ctx_min = 0, ctx_max = 0, window_batches = 0;
		bool timing = false;
		auto launch = [&](const ScheduledBatch &batch, int parity) {
			Step s;
			cudaEventCreate(&s.start); cudaEventCreate(&s.end);
			bool decode_step = batch.phase == ExecutionPhase::DECODE;
			if (!decode_step)
				for (size_t b = 0; b < batch.plan.req_ids.size(); ++b)
					if (batch.plan.starts[b] + batch.plan.lens[b] == P) ++prompts_done;
			bool steady = decode_step && prompts_done == B && scheduler.num_prefill() == 0;
			s.timed = steady && timing;
			cudaEventRecord(s.start, llm.stream());
			llm.inference(batch, parity, engine, buffers);
			cudaEventRecord(s.end, llm.stream());
			steps.push_back(s);
			if (steady) steady_tokens += (long)batch.plan.req_ids.size();
			if (s.timed) {
				window_tokens += (long)batch.plan.req_ids.size();
				++window_batches;
				window_h2d += h2d_bytes((int)batch.plan.req_ids.size(), (int)batch.plan.ids.size());
				for (int start : batch.plan.starts) {ctx_min = ctx_min ? std::min(ctx_min, start + 1) : start + 1; ctx_max = std::max(ctx_max, start + 1);}
			}
		};
		int finished = 0;
		auto on_finished = [&](std::vector<Request> &&done) {finished += (int)done.size();};
		double wall_ms = 0;
		bool ok = true;
		{
			PipelineDriver driver(scheduler, buffers.h_tokens, buffers.token_stride, llm.stream(), launch, on_finished);
			auto pump_until = [&](long target) {
				int guard = 0;
				while (steady_tokens < target && ok) {
					if (driver.pump() == PipelineDriver::Pump::IDLE || ++guard > 1000000) ok = false;
				}
			};
			pump_until((long)W * B);
			if (ok) {
				long base = steady_tokens;
				timing = true;
				double t0 = now_ms();
				pump_until(base + (long)K * B);
				wall_ms = now_ms() - t0;
				timing = false;
			}
			driver.run_to_idle();
		}
		if (!cuda_ok("decode")) return;
		double busy = 0, span = 0;
		cudaEvent_t first = nullptr, last = nullptr;
		for (Step &s : steps) {
			if (s.timed) {
				float ms; cudaEventElapsedTime(&ms, s.start, s.end);
				busy += ms;
				if (!first) first = s.start;
				last = s.end;
			}
		}
		if (first) {float ms; cudaEventElapsedTime(&ms, first, last); span = ms;}
		for (Step &s : steps) {cudaEventDestroy(s.start); cudaEventDestroy(s.end);}
		if (!ok || window_tokens < (long)K * B) {
			std::printf("{\"mode\": \"decode\", \"error\": \"the schedule did not reach %d steady decode steps (%ld tokens)\"}\n", K, window_tokens);
			return;
		}
		double rounds = window_tokens / (double)B;
		std::printf("{\"mode\": \"decode\", \"batch\": %d, \"prompt_len\": %d, \"warmup\": %d, \"steps\": %d, "
		            "\"ms_per_step\": %.5f, \"ms_per_step_span\": %.5f, \"wall_ms_per_step\": %.5f, "
		            "\"tok_s_device\": %.2f, \"tok_s_e2e\": %.2f, \"h2d_bytes_per_step\": %ld, \"d2h_bytes_per_step\": %ld, "
		            "\"batches_per_step\": %.3f, \"tokens\": %ld, \"ctx_min\": %d, \"ctx_max\": %d, \"finished\": %d, "
		            "\"graphs_decode\": %zu, \"preemptions\": %d}\n",
		            B, P, W, K, busy / rounds, span / rounds, wall_ms / rounds, window_tokens / (busy / 1e3), window_tokens / (wall_ms / 1e3),
		            (long)(window_h2d / rounds + 0.5), 4L * B, window_batches / rounds, window_tokens,
		            ctx_min, ctx_max, finished, llm.num_graphs(ExecutionPhase::DECODE), scheduler.num_preemptions());
	}

	void prefill(int T, int W, int K) {
		if (T > max_tokens || T + 1 > max_seq_len) {
			std::printf("{\"mode\": \"prefill\", \"refused\": \"%d tokens exceed --max-tokens %d or --max-seq-len %d\"}\n", T, max_tokens, max_seq_len);
			return;
		}
		std::vector<double> ms_all, wall_all;
		for (int rep = 0; rep < W + K; ++rep) {
			LocalKvHandoff handoff;
			Scheduler scheduler(pool, {max_seqs, max_tokens, -1}, handoff);
			scheduler.add_request(random_prompt(T), 1);
			cudaEvent_t a, b;
			cudaEventCreate(&a); cudaEventCreate(&b);
			int launches = 0;
			auto launch = [&](const ScheduledBatch &batch, int parity) {
				cudaEventRecord(a, llm.stream());
				llm.inference(batch, parity, engine, buffers);
				cudaEventRecord(b, llm.stream());
				++launches;
			};
			auto on_finished = [&](std::vector<Request> &&) {};
			cudaStreamSynchronize(llm.stream());
			double t0 = now_ms();
			{
				PipelineDriver driver(scheduler, buffers.h_tokens, buffers.token_stride, llm.stream(), launch, on_finished);
				driver.run_to_idle();
			}
			double wall = now_ms() - t0;
			if (!cuda_ok("prefill")) return;
			float ms; cudaEventElapsedTime(&ms, a, b);
			cudaEventDestroy(a); cudaEventDestroy(b);
			if (launches != 1) {
				std::printf("{\"mode\": \"prefill\", \"error\": \"%d steps instead of one\"}\n", launches);
				return;
			}
			if (rep >= W) {ms_all.push_back(ms); wall_all.push_back(wall);}
		}
		std::sort(ms_all.begin(), ms_all.end());
		std::sort(wall_all.begin(), wall_all.end());
		double med = ms_all[ms_all.size() / 2], wmed = wall_all[wall_all.size() / 2];
		std::printf("{\"mode\": \"prefill\", \"tokens\": %d, \"ms\": %.4f, \"wall_ms\": %.4f, \"tok_s\": %.1f, \"reps\": %zu, "
		            "\"note\": \"the reference runs its LM head on every row (model/modules/LMHead.h)\"}\n",
		            T, med, wmed, T / (med / 1e3), ms_all.size());
	}

	// the reference's own end-to-end benchmark (model/llm/test/bench_tiny_llama_load.cu:105-160)
	void load(int R, int P, int N) {
		if (P > max_seq_len - N) {std::printf("{\"mode\": \"load\", \"refused\": \"too long\"}\n"); return;}
		double wall = 0, busy = 0, gap = 0;
		int steps_n = 0, finished = 0;
		for (int pass = 0; pass < 2; ++pass) {                  // a short pass first, as the reference does
			int requests = pass ? R : std::min(R, max_seqs), prompt = pass ? P : 16, fresh = pass ? N : 4;
			LocalKvHandoff handoff;
			Scheduler scheduler(pool, {max_seqs, max_tokens, -1}, handoff);
			for (int r = 0; r < requests; ++r) scheduler.add_request(random_prompt(prompt), fresh);
			std::vector<Step> steps;
			steps.reserve(requests * (fresh + 2) + 16);
			auto launch = [&](const ScheduledBatch &batch, int parity) {
				Step s; s.timed = true;
				cudaEventCreate(&s.start); cudaEventCreate(&s.end);
				cudaEventRecord(s.start, llm.stream());
				llm.inference(batch, parity, engine, buffers);
				cudaEventRecord(s.end, llm.stream());
				steps.push_back(s);
			};
			finished = 0;
			auto on_finished = [&](std::vector<Request> &&done) {finished += (int)done.size();};
			cudaStreamSynchronize(llm.stream());
			double t0 = now_ms();
			{
				PipelineDriver driver(scheduler, buffers.h_tokens, buffers.token_stride, llm.stream(), launch, on_finished);
				driver.run_to_idle();
			}
			wall = now_ms() - t0;
			if (!cuda_ok("load")) return;
			busy = gap = 0;
			for (size_t i = 0; i < steps.size(); ++i) {
				float ms; cudaEventElapsedTime(&ms, steps[i].start, steps[i].end); busy += ms;
				if (i) {cudaEventElapsedTime(&ms, steps[i - 1].end, steps[i].start); gap += ms;}
			}
			steps_n = (int)steps.size();
			for (Step &s : steps) {cudaEventDestroy(s.start); cudaEventDestroy(s.end);}
		}
		std::printf("{\"mode\": \"load\", \"requests\": %d, \"prompt_len\": %d, \"new_tokens\": %d, \"max_seqs\": %d, "
		            "\"wall_s\": %.4f, \"tok_s\": %.2f, \"steps\": %d, \"gpu_busy_ms\": %.3f, \"gpu_gap_ms\": %.3f, \"finished\": %d}\n",
		            R, P, N, max_seqs, wall / 1e3, R * (double)N / (wall / 1e3), steps_n, busy, gap, finished);
	}

	void dump_logits(const std::string &path, const std::vector<int> &prompt) {
		int n = (int)prompt.size();
		if (n == 0 || n > max_tokens || n + 1 > max_seq_len) {std::printf("{\"mode\": \"logits\", \"refused\": \"prompt length\"}\n"); return;}
		for (int t : prompt) if (t < 0 || t >= VOCAB) {std::printf("{\"mode\": \"logits\", \"refused\": \"token id\"}\n"); return;}
		LocalKvHandoff handoff;
		Scheduler scheduler(pool, {max_seqs, max_tokens, -1}, handoff);
		scheduler.add_request(prompt, 1);
		int token = -1;
		auto launch = [&](const ScheduledBatch &batch, int parity) {llm.inference(batch, parity, engine, buffers);};
		auto on_finished = [&](std::vector<Request> &&done) {for (Request &r : done) token = r.token_ids.back();};
		{
			PipelineDriver driver(scheduler, buffers.h_tokens, buffers.token_stride, llm.stream(), launch, on_finished);
			driver.run_to_idle();
		}
		if (!cuda_ok("logits")) return;
		std::vector<__nv_bfloat16> row(VOCAB);
		cudaMemcpy(row.data(), static_cast<const __nv_bfloat16 *>(logits->ptr) + (size_t)(n - 1) * VOCAB,
		           VOCAB * sizeof(__nv_bfloat16), cudaMemcpyDeviceToHost);
		std::vector<float> out(VOCAB);
		for (int v = 0; v < VOCAB; ++v) out[v] = __bfloat162float(row[v]);
		FILE *f = std::fopen(path.c_str(), "wb");
		if (!f) {std::printf("{\"mode\": \"logits\", \"error\": \"cannot write %s\"}\n", path.c_str()); return;}
		std::fwrite(out.data(), sizeof(float), out.size(), f);
		std::fclose(f);
		std::printf("{\"mode\": \"logits\", \"tokens\": %d, \"next_token\": %d, \"file\": \"%s\"}\n", n, token, path.c_str());
	}
};

int main(int argc, char **argv) {
	using T = __nv_bfloat16;
	std::string weights;
	int max_seqs = 8, max_seq_len = 2048, layers = 22;
	for (int i = 1; i + 1 < argc; i += 2) {
		std::string k = argv[i], v = argv[i + 1];
		if (k == "--weights") weights = v;
		else if (k == "--max-seqs") max_seqs = std::atoi(v.c_str());
		else if (k == "--max-tokens") g_max_tokens = std::atoi(v.c_str());
		else if (k == "--max-seq-len") max_seq_len = std::atoi(v.c_str());
		else if (k == "--layers") layers = std::atoi(v.c_str());
		else {std::fprintf(stderr, "unknown option %s\n", k.c_str()); return 2;}
	}
	if (weights.empty() || max_seqs < 1 || g_max_tokens < max_seqs || layers < 1 || layers > 22) {
		std::fprintf(stderr, "usage: ref_harness --weights model.safetensors [--max-seqs S] [--max-tokens T] [--max-seq-len L] [--layers N]\n");
		return 2;
	}
	cudaDeviceProp device;
	if (cudaGetDeviceProperties(&device, 0) != cudaSuccess) {std::fprintf(stderr, "no CUDA device\n"); return 3;}

	LLM llm(512);
	Engine engine(llm.arena(), NH, NKV, HS, max_seqs, max_seq_len, g_max_tokens);
	Tensor *token_ids = llm.arena().alloc({g_max_tokens}, Dtype::I32);
	Embedding<T> embedding(llm, token_ids, g_max_tokens, VOCAB, HIDDEN, "model.embed_tokens");
	std::vector<std::unique_ptr<Block<T>>> blocks;
	blocks.reserve(layers);
	Tensor *hidden = embedding.out();
	for (int layer = 0; layer < layers; ++layer) {
		blocks.emplace_back(std::make_unique<Block<T>>(llm, engine, hidden, layer));
		hidden = blocks.back()->out();
	}
	RMSNorm<T> final_norm(llm, hidden, g_max_tokens, HIDDEN, RMS_EPS, "model.norm");
	LMHead<T> lm_head(llm, final_norm.out(), g_max_tokens, HIDDEN, VOCAB, "lm_head");
	llm.finalize();
	KVAlloc kv = llm.arena().alloc_kv_pool();
	KV_Pool pool(kv.k_base, kv.v_base, Dtype::BF16, NKV * HS, kv.bytes_each, layers, max_seqs, max_seq_len);
	engine.bind_pool(&pool);
	engine.init_rope(llm.stream(), ROPE_THETA);
	double t0 = now_ms();
	try {
		llm.load_safetensor(weights, [](const std::string &name) {
			return name == "lm_head.weight" || name.find("_proj.weight") != std::string::npos;
		});
	} catch (const std::exception &e) {
		std::printf("{\"error\": \"load_safetensor: %s\"}\n", e.what());
		return 4;
	}
	if (!cuda_ok("load_safetensor")) return 4;
	std::printf("{\"mode\": \"ready\", \"device\": \"%s\", \"sms\": %d, \"layers\": %d, \"max_seqs\": %d, \"max_tokens\": %d, "
	            "\"max_seq_len\": %d, \"kv_blocks\": %zu, \"load_s\": %.1f}\n", device.name, device.multiProcessorCount, layers,
	            max_seqs, g_max_tokens, max_seq_len, pool.num_free_blocks(), (now_ms() - t0) / 1e3);
	std::fflush(stdout);

	Harness h(llm, engine, pool, lm_head.out(), max_seqs, g_max_tokens, max_seq_len);
	std::string line;
	while (std::getline(std::cin, line)) {
		std::istringstream in(line);
		std::string cmd;
		if (!(in >> cmd)) continue;
		if (cmd == "decode") {int B, P, W, K; if (in >> B >> P >> W >> K) h.decode(B, P, W, K);}
		else if (cmd == "prefill") {int T2, W, K; if (in >> T2 >> W >> K) h.prefill(T2, W, K);}
		else if (cmd == "load") {int R, P, N; if (in >> R >> P >> N) h.load(R, P, N);}
		else if (cmd == "logits") {
			std::string path; std::vector<int> prompt; int t;
			in >> path;
			while (in >> t) prompt.push_back(t);
			h.dump_logits(path, prompt);
		}
		else std::printf("{\"error\": \"unknown command %s\"}\n", cmd.c_str());
		std::fflush(stdout);
		if (cudaPeekAtLastError() != cudaSuccess) return 5;
	}
	return 0;
}
