/*
 * gtest.h -- a minimal stand-in for GoogleTest, just large enough for minml's own test files to compile UNCHANGED
 * (they use TEST, EXPECT_{EQ,NE,LT,LE,TRUE,FALSE,THROW}, GTEST_SKIP, GTEST_SKIP_, ::testing::InitGoogleTest, RUN_ALL_TESTS).
 * GoogleTest itself is not installed on the build machine.  The runner prints one line per test
 *     [ OK | FAILED | SKIPPED ] Suite.name
 * and a final JSON summary; `--gtest_filter=<pattern>[:<pattern>...]` with `*` wildcards selects tests, a leading '-'
 * section excludes.  A test that throws counts as failed.
 */
#pragma once

#include <cstdio>
#include <cstring>
#include <exception>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

namespace testing
{
	struct TestInfo
	{
			const char *suite;
			const char *name;
			void (*body)();
	};
	inline std::vector<TestInfo>& registry()
	{
		static std::vector<TestInfo> tests;
		return tests;
	}
	struct Registrar
	{
			Registrar(const char *suite, const char *name, void (*body)())
			{
				registry().push_back(TestInfo { suite, name, body });
			}
	};
	struct State
	{
			int failures = 0;
			bool skipped = false;
			std::string filter = "*";
	};
	inline State& state()
	{
		static State s;
		return s;
	}
	/* Collects an optional `<< message` after a macro and reports on destruction. */
	class Reporter
	{
			std::ostringstream m_text;
			bool m_failed;
		public:
			Reporter(bool failed, const char *file, int line, const std::string &what) :
					m_failed(failed)
			{
				if (failed)
				{
					state().failures++;
					m_text << file << ":" << line << ": " << what << " ";
				}
			}
			~Reporter()
			{
				if (m_failed)
					std::cout << "    " << m_text.str() << std::endl;
			}
			template<typename T>
			Reporter& operator<<(const T &x)
			{
				if (m_failed)
					m_text << x;
				return *this;
			}
	};
	template<typename A, typename B>
	std::string describe(const char *op, const char *ea, const char *eb, const A &a, const B &b)
	{
		std::ostringstream os;
		os << "expected " << ea << " " << op << " " << eb << " (" << a << " vs " << b << ")";
		return os.str();
	}
	inline bool wildcard_match(const char *pattern, const char *text)
	{
		if (*pattern == '\0')
			return *text == '\0';
		if (*pattern == '*')
			return wildcard_match(pattern + 1, text) || (*text != '\0' && wildcard_match(pattern, text + 1));
		return *text != '\0' && (*pattern == '?' || *pattern == *text) && wildcard_match(pattern + 1, text + 1);
	}
	inline bool selected(const std::string &full_name)
	{
		std::string positive = state().filter, negative;
		const size_t dash = positive.find('-');
		if (dash != std::string::npos)
		{
			negative = positive.substr(dash + 1);
			positive = positive.substr(0, dash);
		}
		if (positive.empty())
			positive = "*";
		auto any = [&](const std::string &list)
		{
			size_t start = 0;
			while (start <= list.size())
			{
				size_t end = list.find(':', start);
				if (end == std::string::npos)
					end = list.size();
				const std::string pat = list.substr(start, end - start);
				if (!pat.empty() && wildcard_match(pat.c_str(), full_name.c_str()))
					return true;
				start = end + 1;
			}
			return false;
		};
		return any(positive) && !(negative.size() > 0 && any(negative));
	}
	inline void InitGoogleTest(int *argc, char **argv)
	{
		for (int i = 1; i < *argc; i++)
			if (std::strncmp(argv[i], "--gtest_filter=", 15) == 0)
				state().filter = argv[i] + 15;
	}
	inline int run_all()
	{
		int passed = 0, failed = 0, skipped = 0;
		std::vector<std::string> failed_names;
		for (const TestInfo &t : registry())
		{
			const std::string full = std::string(t.suite) + "." + t.name;
			if (!selected(full))
				continue;
			state().failures = 0;
			state().skipped = false;
			try
			{
				t.body();
			}
			catch (const std::exception &e)
			{
				state().failures++;
				std::cout << "    uncaught exception: " << e.what() << std::endl;
			}
			catch (...)
			{
				state().failures++;
				std::cout << "    uncaught exception" << std::endl;
			}
			if (state().failures > 0)
			{
				failed++;
				failed_names.push_back(full);
				std::cout << "[ FAILED  ] " << full << std::endl;
			}
			else if (state().skipped)
			{
				skipped++;
				std::cout << "[ SKIPPED ] " << full << std::endl;
			}
			else
			{
				passed++;
				std::cout << "[ OK      ] " << full << std::endl;
			}
		}
		std::cout << "{\"passed\": " << passed << ", \"failed\": " << failed << ", \"skipped\": " << skipped << ", \"failed_tests\": [";
		for (size_t i = 0; i < failed_names.size(); i++)
			std::cout << (i ? ", " : "") << "\"" << failed_names[i] << "\"";
		std::cout << "]}" << std::endl;
		return failed == 0 ? 0 : 1;
	}
} /* namespace testing */

#define TEST(suite, name) \
	static void suite##_##name##_body(); \
	static ::testing::Registrar suite##_##name##_registrar(#suite, #name, &suite##_##name##_body); \
	static void suite##_##name##_body()

#define GTEST_COMPARE_(a, b, op) ::testing::Reporter(!((a) op (b)), __FILE__, __LINE__, ::testing::describe(#op, #a, #b, (a), (b)))
#define EXPECT_EQ(a, b) GTEST_COMPARE_(a, b, ==)
#define EXPECT_NE(a, b) GTEST_COMPARE_(a, b, !=)
#define EXPECT_LT(a, b) GTEST_COMPARE_(a, b, <)
#define EXPECT_LE(a, b) GTEST_COMPARE_(a, b, <=)
#define EXPECT_GT(a, b) GTEST_COMPARE_(a, b, >)
#define EXPECT_GE(a, b) GTEST_COMPARE_(a, b, >=)
#define EXPECT_TRUE(x) ::testing::Reporter(!static_cast<bool>(x), __FILE__, __LINE__, "expected true: " #x)
#define EXPECT_FALSE(x) ::testing::Reporter(static_cast<bool>(x), __FILE__, __LINE__, "expected false: " #x)
#define EXPECT_THROW(statement, exception_type) \
	do { \
		bool gtest_caught = false; \
		try { statement; } catch (const exception_type&) { gtest_caught = true; } catch (...) { } \
		::testing::Reporter(!gtest_caught, __FILE__, __LINE__, "expected " #statement " to throw " #exception_type); \
	} while (0)
#define GTEST_SKIP() do { ::testing::state().skipped = true; return; } while (0)
#define GTEST_SKIP_(message) do { ::testing::state().skipped = true; return; } while (0)
#define RUN_ALL_TESTS() ::testing::run_all()
