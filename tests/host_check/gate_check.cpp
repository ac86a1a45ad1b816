// TEST PROGRAM for the start gate of the multi-GPU driver (clpeak_b200/csrc/host/start_gate.hpp):
// all parties meet; a missing party breaks the gate after the timeout instead of hanging the
// others; a party that leaves no longer counts.  Prints one line per check; exit code = failures.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <thread>
#include <vector>

#include "start_gate.hpp"

static int g_failed = 0;
static void report(const char *what, bool ok)
{
    std::printf("%-58s %s\n", what, ok ? "ok" : "FAILED");
    if (!ok)
        ++g_failed;
}

int main()
{
    using ms = std::chrono::milliseconds;
    {   // three parties, five rounds: nobody passes a round before the last one arrives
        StartGate gate(3);
        std::atomic<int> arrived{0}, early{0}, met{0};
        std::vector<std::thread> ts;
        for (int t = 0; t < 3; ++t)
            ts.emplace_back([&, t] {
                for (int round = 0; round < 5; ++round) {
                    std::this_thread::sleep_for(ms(5 * t));
                    ++arrived;
                    if (gate.arrive(ms(5000)))
                        ++met;
                    if (arrived.load() < 3 * (round + 1))
                        ++early;
                }
            });
        for (auto &t : ts)
            t.join();
        report("three parties meet in every round", met == 15 && early == 0 && !gate.broken());
    }
    {   // one party never arrives: the others give up after the timeout, later arrivals do not wait
        StartGate gate(3);
        std::atomic<int> met{0};
        const auto t0 = std::chrono::steady_clock::now();
        std::thread a([&] { met += gate.arrive(ms(150)) ? 1 : 0; });
        std::thread b([&] { met += gate.arrive(ms(150)) ? 1 : 0; });
        a.join();
        b.join();
        const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        const auto t1 = std::chrono::steady_clock::now();
        const bool again = gate.arrive(ms(5000));
        const double second = std::chrono::duration<double>(std::chrono::steady_clock::now() - t1).count();
        report("a missing party breaks the gate after the timeout", met == 0 && gate.broken() && waited >= 0.14 && waited < 3.0);
        report("a broken gate no longer blocks", !again && second < 0.5);
    }
    {   // a party that leaves is no longer waited for
        StartGate gate(3);
        std::atomic<int> met{0};
        std::thread a([&] { met += gate.arrive(ms(5000)) ? 1 : 0; });
        std::thread b([&] { met += gate.arrive(ms(5000)) ? 1 : 0; });
        std::this_thread::sleep_for(ms(50));
        gate.leave();
        a.join();
        b.join();
        report("leave() releases the parties that were waiting", met == 2 && !gate.broken());
        std::thread c([&] { met += gate.arrive(ms(5000)) ? 1 : 0; });
        std::thread d([&] { met += gate.arrive(ms(5000)) ? 1 : 0; });
        c.join();
        d.join();
        report("the remaining two parties keep meeting", met == 4 && !gate.broken());
    }
    {   // a single party never waits
        StartGate gate(1);
        report("a lone party passes at once", gate.arrive(ms(5000)) && !gate.broken());
    }
    return g_failed;
}
