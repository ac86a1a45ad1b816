// The scoped logger: backends open backend / device / test scopes and emit
// readings; the base class keeps the result table and the device table and
// hands every moment to one virtual hook as a LogEvent.  Behaviour follows the
// reference (src/common/logger.cpp): at most one test open at a time, a stale
// TestScope never closes somebody else's test, device rows are de-duplicated by
// (backend, platform, device, driver), free text is folded to one line.
#include <cassert>
#include <cctype>
#include <cmath>
#include <iomanip>
#include <sstream>

#include "clpeak_api.hpp"

namespace {

// Descriptions are authored as multi-line C++ string literals; fold every run of
// whitespace into one blank so they survive the XML attribute / CSV cell.
std::string foldWhitespace(const std::string &text)
{
    std::istringstream words(text);
    std::string out, w;
    while (words >> w) {
        if (!out.empty())
            out.push_back(' ');
        out += w;
    }
    return out;
}

} // namespace

logger::logger(std::string compareFileName) : compareEnabled(!compareFileName.empty())
{
    if (compareEnabled)
        baseline = buildBaselineMap(loadResultFile(compareFileName));
}

LogEvent logger::makeEvent(LogEvent::Kind kind) const
{
    LogEvent ev;
    ev.kind = kind;
    ev.backend = curBackend;
    ev.platform = curPlatform;
    ev.device = curDevice;
    ev.driver = curDriver;
    ev.testTag = curTest;
    ev.testDisplay = curTestDisplay;
    ev.testDescription = curTestDescription;
    ev.unit = curUnit;
    ev.category = curCategory;
    return ev;
}

ResultEntry logger::makeEntry(const std::string &metric, ResultStatus status, float value,
                              const std::string &reason, const std::string &metricDescription) const
{
    ResultEntry row;
    row.backend = curBackend;
    row.platform = curPlatform;
    row.device = curDevice;
    row.driver = curDriver;
    row.category = categoryString(curCategory);
    row.test = curTest;
    row.metric = metric;
    row.unit = curUnit;
    row.status = status;
    row.value = value;
    row.reason = reason;
    row.display = curTestDisplay;
    row.description = curTestDescription;
    row.metricDescription = foldWhitespace(metricDescription);
    return row;
}

void logger::note(const std::string &msg)
{
    LogEvent ev = makeEvent(LogEvent::Kind::Note);
    ev.message = msg;
    onEvent(ev);
}

logger::BackendScope logger::beginBackend(const std::string &name) { return BackendScope(this, name); }

// ---- backend scope --------------------------------------------------------

logger::BackendScope::BackendScope(logger *l, const std::string &name) : log(l)
{
    assert(log->contextDepth == 0);
    log->curBackend = name;
    log->curPlatform.clear();
    log->curDevice.clear();
    log->curDriver.clear();
    log->contextDepth = 1;
    log->onEvent(log->makeEvent(LogEvent::Kind::BackendBegin));
}

logger::BackendScope::BackendScope(BackendScope &&o) noexcept : log(o.log), closed(o.closed)
{
    o.log = nullptr;
    o.closed = true;
}

logger::BackendScope::~BackendScope() { end(); }

void logger::BackendScope::end()
{
    if (closed)
        return;
    closed = true;
    log->onEvent(log->makeEvent(LogEvent::Kind::BackendEnd));
    log->curBackend.clear();
    log->contextDepth = 0;
}

logger::DeviceScope logger::BackendScope::beginDevice(const DeviceSpec &spec)
{
    assert(!closed && log->contextDepth == 1);
    return DeviceScope(log, spec);
}

// ---- device scope ----------------------------------------------------------

logger::DeviceScope::DeviceScope(logger *l, const DeviceSpec &spec) : log(l)
{
    log->curPlatform = spec.platform.empty() ? log->curBackend : spec.platform;
    log->curDevice = spec.name;
    log->curDriver = spec.driver_version;
    log->contextDepth = 2;

    DeviceInfo info{log->curBackend, log->curPlatform, log->curDevice, log->curDriver, spec.props};
    auto it = std::find_if(log->devices.begin(), log->devices.end(),
                           [&](const DeviceInfo &d) { return d.key() == info.key(); });
    if (it == log->devices.end())
        log->devices.push_back(info);
    else
        it->props = info.props;

    LogEvent ev = log->makeEvent(LogEvent::Kind::DeviceBegin);
    ev.props = spec.props;
    ev.platformIndex = spec.platform_index;
    ev.deviceIndex = spec.device_index;
    ev.showPlatformLine = (log->curPlatform != log->curBackend);
    log->onEvent(ev);
}

logger::DeviceScope::DeviceScope(DeviceScope &&o) noexcept : log(o.log), closed(o.closed)
{
    o.log = nullptr;
    o.closed = true;
}

logger::DeviceScope::~DeviceScope() { end(); }

void logger::DeviceScope::end()
{
    if (closed)
        return;
    closed = true;
    log->closeOpenTest();
    log->onEvent(log->makeEvent(LogEvent::Kind::DeviceEnd));
    log->curDevice.clear();
    log->curDriver.clear();
    log->curPlatform.clear();
    log->contextDepth = 1;
}

void logger::closeOpenTest()
{
    if (contextDepth != 3)
        return;
    onEvent(makeEvent(LogEvent::Kind::TestEnd));
    curTest.clear();
    curTestDisplay.clear();
    curTestDescription.clear();
    curUnit.clear();
    curCategory = Category::Unknown;
    curTestSeq = 0;
    contextDepth = 2;
}

logger::TestScope logger::DeviceScope::beginTest(const TestSpec &spec)
{
    assert(!closed);
    if (log->contextDepth == 3) {
        const std::string previous = log->curTest;
        log->closeOpenTest();
        log->note("logger: test '" + spec.tag + "' opened while '" + previous +
                  "' was still open; closed it first");
    }
    return TestScope(log, spec);
}

// ---- test scope ------------------------------------------------------------

logger::TestScope::TestScope(logger *l, const TestSpec &spec) : log(l)
{
    log->curTest = spec.tag;
    log->curTestDisplay = spec.display;
    log->curTestDescription = foldWhitespace(spec.description);
    log->curUnit = spec.unit;
    log->curCategory = spec.category != Category::Unknown ? spec.category : categoryFromUnit(spec.unit);
    log->contextDepth = 3;
    seq = ++log->testSeqCounter;
    log->curTestSeq = seq;
    log->onEvent(log->makeEvent(LogEvent::Kind::TestBegin));
}

logger::TestScope::TestScope(TestScope &&o) noexcept : log(o.log), closed(o.closed), seq(o.seq)
{
    o.log = nullptr;
    o.closed = true;
}

logger::TestScope::~TestScope() { end(); }

void logger::TestScope::emit(std::string metric, float value, EmitOptions opts)
{
    assert(!closed && log->contextDepth == 3);
    LogEvent ev = log->makeEvent(LogEvent::Kind::Metric);
    ev.entry = log->makeEntry(metric, ResultStatus::Ok, value, "", opts.description);
    ev.subMetric = opts.subMetric;
    log->results.push_back(ev.entry);
    log->onEvent(ev);
}

void logger::TestScope::emit(std::string metric, float value, const char *description)
{
    EmitOptions o;
    if (description)
        o.description = description;
    emit(std::move(metric), value, std::move(o));
}

void logger::TestScope::skip(std::string metric, ResultStatus status, std::string reason, std::string description)
{
    assert(!closed && log->contextDepth == 3);
    LogEvent ev = log->makeEvent(LogEvent::Kind::Metric);
    ev.entry = log->makeEntry(metric, status, 0.0f, reason, description);
    log->results.push_back(ev.entry);
    log->onEvent(ev);
}

void logger::TestScope::skipAll(std::initializer_list<std::string> metrics, ResultStatus status, std::string reason)
{
    assert(!closed && log->contextDepth == 3);
    LogEvent ev = log->makeEvent(LogEvent::Kind::TestSkippedAll);
    ev.status = status;
    ev.reason = reason;
    for (const std::string &m : metrics) {
        log->results.push_back(log->makeEntry(m, status, 0.0f, reason));
        ev.metricNames.push_back(m);
    }
    log->onEvent(ev);
}

void logger::TestScope::end()
{
    if (closed)
        return;
    closed = true;
    if (log->curTestSeq == seq)      // otherwise somebody already closed it
        log->closeOpenTest();
}

// ===========================================================================
// Text channel
// ===========================================================================
//
// Layout (two blanks per level), as the reference CLI prints it
// (src/common/logger_text.cpp):
//   Backend: CUDA
//     Device 0: NVIDIA B200
//       SMs              : 148
//
//       Global memory bandwidth (GBPS)
//         float4   : 6587.83

namespace {
constexpr int kMinPad = 8;
constexpr int kPropPad = 16;
constexpr int kWrapWidth = 100;
constexpr int kMinWrap = 30;

std::string statusLabel(ResultStatus s)
{
    switch (s) {
    case ResultStatus::Unsupported: return "unsupported";
    case ResultStatus::Skipped: return "skipped";
    case ResultStatus::Error: return "error";
    default: return "ok";
    }
}

std::string pad(int level) { return std::string((size_t)std::max(level, 0) * 2, ' '); }
} // namespace

void LoggerText::onEvent(const LogEvent &e)
{
    switch (e.kind) {
    case LogEvent::Kind::BackendBegin:
        out << "\nBackend: " << e.backend << "\n";
        depth = 1;
        break;
    case LogEvent::Kind::DeviceBegin: {
        int lvl = 1;
        if (e.showPlatformLine) {
            out << pad(lvl) << "Platform" << (e.platformIndex >= 0 ? " " + std::to_string(e.platformIndex) : "")
                << ": " << e.platform << "\n";
            lvl++;
        }
        out << pad(lvl) << "Device" << (e.deviceIndex >= 0 ? " " + std::to_string(e.deviceIndex) : "") << ": "
            << e.device << "\n";
        propDepth = lvl + 1;
        metricDepth = propDepth + 1;
        if (!e.driver.empty()) {
            std::string k = "Driver version";
            k.resize(std::max<size_t>(k.size(), kPropPad), ' ');
            out << pad(propDepth) << k << " : " << e.driver << "\n";
        }
        for (const auto &p : e.props) {
            std::string k = p.key;
            k.resize(std::max<size_t>(k.size(), kPropPad), ' ');
            out << pad(propDepth) << k << " : " << p.value << "\n";
        }
        out << "\n";
        depth = propDepth;
        out.flush();
        break;
    }
    case LogEvent::Kind::TestBegin: {
        std::string head = e.testDisplay;
        if (!e.unit.empty()) {
            std::string u = e.unit;
            for (auto &c : u)
                c = (char)std::toupper((unsigned char)c);
            head += " (" + u + ")";
        }
        out << pad(propDepth) << head << "\n";
        if (describe && !e.testDescription.empty()) {
            wrapText(metricDepth * 2, e.testDescription);
            out << "\n";
        }
        rows.clear();
        out.flush();
        break;
    }
    case LogEvent::Kind::Metric:
        rows.push_back({e.entry.metric, e.entry.value, e.entry.status, e.entry.reason, e.subMetric, e.entry.key(),
                        e.entry.metricDescription});
        break;
    case LogEvent::Kind::TestSkippedAll:
        out << pad(metricDepth) << "[" << statusLabel(e.status) << "] " << e.reason << "\n";
        out.flush();
        break;
    case LogEvent::Kind::TestEnd:
        flushRows();
        out << "\n";
        break;
    case LogEvent::Kind::DeviceEnd:
        flushRows();
        depth = 1;
        out.flush();
        break;
    case LogEvent::Kind::BackendEnd:
        depth = 0;
        out.flush();
        break;
    case LogEvent::Kind::Note:
        out << pad(depth) << e.message;
        if (e.message.empty() || e.message.back() != '\n')
            out << "\n";
        out.flush();
        break;
    }
}

void LoggerText::flushRows()
{
    if (rows.empty())
        return;
    int width = kMinPad;
    for (const auto &r : rows)
        width = std::max(width, (int)r.metric.size());
    for (const auto &r : rows) {
        const int lvl = r.sub ? metricDepth + 1 : metricDepth;
        const int target = std::max(kMinPad, r.sub ? width - 2 : width);
        std::string name = r.metric;
        if ((int)name.size() < target)
            name.resize((size_t)target, ' ');
        out << pad(lvl) << name << " : ";
        if (r.status == ResultStatus::Ok) {
            std::ostringstream v;
            v << std::fixed << std::setprecision(2) << r.value;
            out << v.str();
            if (compareEnabled) {
                auto it = baseline.find(r.key);
                if (it != baseline.end()) {
                    const float base = it->second;
                    const float delta = base != 0.0f ? 100.0f * (r.value - base) / base : 0.0f;
                    std::ostringstream d;
                    d << "  (was " << std::fixed << std::setprecision(2) << base << ", " << (delta >= 0 ? '+' : '-')
                      << std::setprecision(1) << std::fabs(delta) << "%)";
                    out << d.str();
                }
            }
            out << "\n";
        } else {
            out << "[" << statusLabel(r.status) << "] " << r.reason << "\n";
        }
        if (describe && !r.info.empty())
            wrapText(lvl * 2 + target + 3, r.info);
    }
    rows.clear();
    out.flush();
}

void LoggerText::wrapText(int column, const std::string &text)
{
    column = std::max(column, 0);
    const int width = std::max(kMinWrap, kWrapWidth - column);
    const std::string indent((size_t)column, ' ');
    std::istringstream words(text);
    std::string line, w;
    while (words >> w) {
        if (!line.empty() && (int)(line.size() + 1 + w.size()) > width) {
            out << indent << line << "\n";
            line.clear();
        }
        if (!line.empty())
            line.push_back(' ');
        line += w;
    }
    if (!line.empty())
        out << indent << line << "\n";
}
