// The clpeak_ffi exports (include/clpeak_ffi.h) and the JSON event channel.
//
// Behaviour restated from the reference (src/ffi/clpeak_ffi.cpp:164-225,
// src/ffi/logger_ffi.cpp:54-141): one launch at a time (BUSY without a done
// event otherwise), bad argv -> note + done + BAD_ARGS, result files written
// even after a cancel, `done` always last, every event string malloc'd and
// owned by the callee, numbers printed in the classic locale.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <iomanip>
#include <locale>
#include <sstream>

#include <cuda/cuda_peak.h>
#include <common/options.h>

#include "../../../include/clpeak_ffi.h"
#include "backend_table.hpp"

namespace {

char *mallocCopy(const std::string &s)
{
    char *p = static_cast<char *>(std::malloc(s.size() + 1));
    if (p)
        std::memcpy(p, s.c_str(), s.size() + 1);
    return p;
}

const char *kindName(LogEvent::Kind k)
{
    switch (k) {
    case LogEvent::Kind::BackendBegin: return "backend_begin";
    case LogEvent::Kind::DeviceBegin: return "device";
    case LogEvent::Kind::TestBegin: return "test_begin";
    case LogEvent::Kind::Metric: return "metric";
    case LogEvent::Kind::TestSkippedAll: return "test_skipped";
    case LogEvent::Kind::TestEnd: return "test_end";
    case LogEvent::Kind::DeviceEnd: return "device_end";
    case LogEvent::Kind::BackendEnd: return "backend_end";
    case LogEvent::Kind::Note: return "note";
    }
    return "unknown";
}

class JsonObject {
public:
    JsonObject() { ss_.imbue(std::locale::classic()); ss_ << "{"; }
    JsonObject &str(const char *k, const std::string &v)
    {
        sep();
        ss_ << "\"" << k << "\":\"" << jsonEscape(v) << "\"";
        return *this;
    }
    JsonObject &raw(const char *k, const std::string &v)
    {
        sep();
        ss_ << "\"" << k << "\":" << v;
        return *this;
    }
    std::string done() { ss_ << "}"; return ss_.str(); }

private:
    void sep() { if (!first_) ss_ << ","; first_ = false; }
    std::ostringstream ss_;
    bool first_ = true;
};

std::string fixed4(float v)
{
    std::ostringstream ss;
    ss.imbue(std::locale::classic());
    ss << std::fixed << std::setprecision(4) << v;
    return ss.str();
}

std::string eventJson(const LogEvent &e)
{
    JsonObject o;
    o.str("t", kindName(e.kind)).str("backend", e.backend).str("platform", e.platform).str("device", e.device)
        .str("driver", e.driver);
    switch (e.kind) {
    case LogEvent::Kind::DeviceBegin: {
        std::string props = "[";
        for (size_t i = 0; i < e.props.size(); ++i)
            props += std::string(i ? "," : "") + "{\"k\":\"" + jsonEscape(e.props[i].key) + "\",\"v\":\"" +
                     jsonEscape(e.props[i].value) + "\"}";
        props += "]";
        o.raw("platform_index", std::to_string(e.platformIndex)).raw("device_index", std::to_string(e.deviceIndex))
            .raw("props", props);
        break;
    }
    case LogEvent::Kind::TestBegin:
        o.str("test", e.testTag).str("display", e.testDisplay).str("unit", e.unit)
            .str("category", categoryString(e.category)).str("desc", e.testDescription);
        break;
    case LogEvent::Kind::Metric:
        o.str("category", e.entry.category).str("test", e.entry.test).str("display", e.testDisplay)
            .str("metric", e.entry.metric).str("unit", e.entry.unit).raw("value", fixed4(e.entry.value))
            .str("status", statusString(e.entry.status)).str("reason", e.entry.reason)
            .raw("sub", e.subMetric ? "true" : "false").str("desc", e.entry.description)
            .str("minfo", e.entry.metricDescription);
        break;
    case LogEvent::Kind::TestSkippedAll: {
        std::string names = "[";
        for (size_t i = 0; i < e.metricNames.size(); ++i)
            names += std::string(i ? "," : "") + "\"" + jsonEscape(e.metricNames[i]) + "\"";
        names += "]";
        o.str("test", e.testTag).str("display", e.testDisplay).str("unit", e.unit)
            .str("category", categoryString(e.category)).str("desc", e.testDescription).raw("metrics", names)
            .str("status", statusString(e.status)).str("reason", e.reason);
        break;
    }
    case LogEvent::Kind::Note:
        o.str("message", e.message);
        break;
    default:
        break;
    }
    return o.done();
}

void deliver(ClpeakEventCallback cb, void *ud, const std::string &json)
{
    if (!cb)
        return;
    if (char *p = mallocCopy(json))
        cb(ud, p);                       // the callee owns p from here on
}

class LoggerFfi : public logger {
public:
    LoggerFfi(ClpeakEventCallback cb, void *ud) : cb_(cb), ud_(ud) {}

protected:
    void onEvent(const LogEvent &e) override { deliver(cb_, ud_, eventJson(e)); }

private:
    ClpeakEventCallback cb_;
    void *ud_;
};

std::atomic<bool> g_busy{false};

void sendDone(ClpeakEventCallback cb, void *ud, int status, bool cancelled)
{
    deliver(cb, ud, std::string("{\"t\":\"done\",\"status\":") + std::to_string(status) + ",\"cancelled\":" +
                        (cancelled ? "true" : "false") + "}");
}

} // namespace

extern "C" {

const char *clpeak_version(void) { return CLPEAK_VERSION_STR; }

char *clpeak_copy_backend_catalog_json(void)
{
    std::vector<BackendInventory> inv;
    for (const auto &b : clpeakBackends())
        inv.push_back(b.enumerate());
    return mallocCopy(inventoryToJson(inv));
}

void clpeak_free_string(char *s) { std::free(s); }

void clpeak_request_cancel(void) { clpeak::requestCancel(); }

char *clpeak_load_result_file_json(const char *path)
{
    if (!path)
        return nullptr;
    DeviceInfoStore devices;
    const ResultStore rows = loadResultFile(path, &devices);
    return rows.empty() ? nullptr : mallocCopy(resultsToJson(rows, devices));
}

int clpeak_launch(int argc, const char **argv, ClpeakEventCallback on_event, void *user_data)
{
    bool idle = false;
    if (!g_busy.compare_exchange_strong(idle, true))
        return CLPEAK_RUN_BUSY;
    clpeak::resetCancel();

    std::vector<char *> args;
    for (int i = 0; i < argc; ++i)
        args.push_back(const_cast<char *>(argv[i]));
    CliOptions opts;
    std::string problem;
    if (!parseCliOptionsNoExit(argc, args.data(), opts, problem)) {
        LogEvent note;
        note.kind = LogEvent::Kind::Note;
        note.message = problem;
        deliver(on_event, user_data, eventJson(note));
        sendDone(on_event, user_data, CLPEAK_RUN_BAD_ARGS, false);
        g_busy.store(false);
        return CLPEAK_RUN_BAD_ARGS;
    }
    clpeak::setVerbose(opts.verbose);

    ResultStore rows;
    DeviceInfoStore devices;
    int status = 0, ran = 0;
    for (const auto &b : clpeakBackends()) {
        if (opts.*(b.skip) || clpeak::cancelRequested())
            continue;
        ++ran;
        std::unique_ptr<Peak> peak = b.create();
        peak->log.reset(new LoggerFfi(on_event, user_data));
        peak->applyOptions(opts);
        status |= peak->runAll();
        rows.insert(rows.end(), peak->log->results.begin(), peak->log->results.end());
        devices.insert(devices.end(), peak->log->devices.begin(), peak->log->devices.end());
    }
    if (opts.namedAbsentBackend) {
        LogEvent note;
        note.kind = LogEvent::Kind::Note;
        note.message = "the native CPU backend is not built into this library (CUDA backend only)";
        deliver(on_event, user_data, eventJson(note));
        if (ran == 0)
            status |= 1;
    }
    if (opts.enableJson && !saveJson(rows, opts.jsonFile, devices)) status |= 1;
    if (opts.enableCsv && !saveCsv(rows, opts.csvFile)) status |= 1;
    if (opts.enableXml && !saveXml(rows, opts.xmlFile, devices)) status |= 1;

    const bool cancelled = clpeak::cancelRequested();
    const int result = cancelled ? CLPEAK_RUN_CANCELLED : status;
    sendDone(on_event, user_data, result, cancelled);
    g_busy.store(false);
    return result;
}

} // extern "C"
